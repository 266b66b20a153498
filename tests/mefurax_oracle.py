"""A plain, slow restatement of the Mefurax design in float64: one function per mechanism, one token at a time, state kept in Python
lists.  It shares no code with the library.

Notation.  x_t is the residual stream of token t (position t, counted from 0 in its sequence); a layer does
    x <- N1(alpha x + mixer(x)),   x <- N2(alpha x + ff(x)),   N(u) = u / sqrt(mean(u^2) + eps) * (1 + w).
Mixer A ("attention"): u = W x + b for q, k, v; a causal filter over time per channel, c_t = sum_j f[:, j] u_(t - taps + 1 + j) (zeros before
the sequence); q and k each divided by their root mean square over ALL their channels and multiplied by a weight per channel;
score(t, s) = scale q_t . k_s - 2^(-8 (h + 1) / H) (t - s); keys s with 0 <= t - s < size.
Mixer B ("attention_2"): u = W x; pairs (2i, 2i + 1) of the first `dims` channels of every head of q and k are rotated by the angle
t base^(-2i / dims); every head of q and k is then divided by its own root mean square; score = cap tanh(scale q . k / cap); keys s <= t
in the same block of `size` positions; head h's output times sigmoid((W_g x)_h).
Both: query head h reads key / value head h // (H / G); layers marked v_mix share values: the first one's v is remembered per token and
every later one uses (1 - l) v + l v_first.  Feed-forward: gated tanh-GELU, or a mixture of relu^2 experts (the `top` largest router
logits, softmax over those) plus an always-on expert."""
import math

import numpy as np


# ------------------------------------------------------------------------------------------------ small pieces
def unit_rms(u, eps):
    return u / math.sqrt(float(np.mean(u * u)) + eps)


def offset_norm(u, w, eps):
    return unit_rms(u, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def filter_step(history, f):
    """history: the projected vectors u_0 .. u_t of this sequence (list); f: [channels, taps].  Returns c_t."""
    taps = f.shape[1]
    t = len(history) - 1
    out = np.zeros(f.shape[0])
    for j in range(taps):
        s = t - taps + 1 + j
        if s >= 0:
            out += f[:, j] * history[s]
    return out


def rotate_pairs(head_vec, pos, dims, base):
    out = head_vec.copy()
    for i in range(dims // 2):
        ang = pos * base ** (-2.0 * i / dims)
        a, b = head_vec[2 * i], head_vec[2 * i + 1]
        out[2 * i] = a * math.cos(ang) - b * math.sin(ang)
        out[2 * i + 1] = b * math.cos(ang) + a * math.sin(ang)
    return out


def sees_window(t, s, size):
    return 0 <= t - s < size


def sees_chunk(t, s, size):
    return s <= t and t // size == s // size


def distance_slope(h, heads):
    return 2.0 ** (-8.0 * (h + 1) / heads)


def soft_cap(score, cap):
    return cap * math.tanh(score / cap)


def softmax(scores):
    e = np.exp(np.asarray(scores) - max(scores))
    return e / e.sum()


def blend(v, v_first, lam):
    return (1.0 - lam) * v + lam * v_first


def expert(h, up, down):
    return down @ (np.maximum(up @ h, 0.0) ** 2)


def route(z, top):
    """Indices of the `top` largest logits (lower index first among equals) and their softmax weights."""
    order = sorted(range(len(z)), key=lambda e: (-z[e], e))[:top]
    return order, softmax([z[e] for e in order])


# ------------------------------------------------------------------------------------------------ the model
class Model:
    def __init__(self, cfg, weights):
        self.cfg = cfg
        self.w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
        self.eps = cfg["norm"]["eps"]
        self.alpha = cfg["postln_alpha"]
        mixing = [i for i, L in enumerate(cfg["layers"]) if L["mixer"].get("v_mix")]
        self.first_mix = mixing[0] if mixing else None

    def new_state(self):
        return {"n": 0, "layers": [{"u": [], "k": [], "v": []} for _ in self.cfg["layers"]]}

    # -- mixers: return the mixer's output for the token at position t and append to the layer's lists
    def mixer_a(self, i, x, t, st, shared):
        m, w, p = self.cfg["layers"][i]["mixer"], self.w, "l%d.mix." % i
        H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        u = np.concatenate([w[p + n] @ x + w[p + n + ".b"] for n in ("q", "k", "v")])
        st["u"].append(u)
        if m.get("conv", 0) > 0:
            f = np.concatenate([w[p + n + ".conv"] for n in ("q", "k", "v")])
            c = filter_step(st["u"], f)
        else:
            c = u
        q, k, v = c[:H * D], c[H * D:(H + G) * D], c[(H + G) * D:]
        q = unit_rms(q, self.eps) * w[p + "q.norm"]
        k = unit_rms(k, self.eps) * w[p + "k.norm"]
        v = self.shared_values(i, v, shared)
        st["k"].append(k.reshape(G, D))
        st["v"].append(v.reshape(G, DV))
        heads = []
        for h in range(H):
            g = h // (H // G)
            seen = [s for s in range(t + 1) if sees_window(t, s, m["mask"]["size"])]
            sc = [m["scale"] * float(q[h * D:(h + 1) * D] @ st["k"][s][g]) - distance_slope(h, H) * (t - s) for s in seen]
            pr = softmax(sc)
            heads.append(sum(pj * st["v"][s][g] for pj, s in zip(pr, seen)))
        return w[p + "o"] @ np.concatenate(heads)

    def mixer_b(self, i, x, t, st, shared):
        m, w, p = self.cfg["layers"][i]["mixer"], self.w, "l%d.mix." % i
        H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        rot = m.get("rot") or {"dims": 0, "base": 1.0}
        q = (w[p + "q"] @ x).reshape(H, D)
        k = (w[p + "k"] @ x).reshape(G, D)
        q = np.stack([unit_rms(rotate_pairs(r, t, rot["dims"], rot["base"]), self.eps) for r in q])
        k = np.stack([unit_rms(rotate_pairs(r, t, rot["dims"], rot["base"]), self.eps) for r in k])
        v = self.shared_values(i, w[p + "v"] @ x, shared)
        st["k"].append(k)
        st["v"].append(v.reshape(G, DV))
        gate = 1.0 / (1.0 + np.exp(-(w[p + "g"] @ x)))
        heads = []
        for h in range(H):
            g = h // (H // G)
            seen = [s for s in range(t + 1) if sees_chunk(t, s, m["mask"]["size"])]
            sc = [m["scale"] * float(q[h] @ st["k"][s][g]) for s in seen]
            if m.get("softcap", 0.0) > 0.0:
                sc = [soft_cap(z, m["softcap"]) for z in sc]
            pr = softmax(sc)
            heads.append(gate[h] * sum(pj * st["v"][s][g] for pj, s in zip(pr, seen)))
        return w[p + "o"] @ np.concatenate(heads)

    def shared_values(self, i, v, shared):
        if not self.cfg["layers"][i]["mixer"].get("v_mix"):
            return v
        if i == self.first_mix:
            shared["v"] = v
            return v
        return blend(v, shared["v"], float(self.w["l%d.mix.vmix" % i]))

    def feed_forward(self, i, h):
        mlp, w, p = self.cfg["layers"][i]["mlp"], self.w, "l%d.mlp." % i
        if mlp["kind"] == "dense":
            return w[p + "down"] @ (gelu_tanh(w[p + "gate"] @ h) * (w[p + "up"] @ h))
        chosen, weights = route(w[p + "router"] @ h, mlp["router"]["top"])
        out = sum(a * expert(h, w[p + "e%d.up" % e], w[p + "e%d.down" % e]) for e, a in zip(chosen, weights))
        if (mlp.get("shared") or {}).get("ff", 0) > 0:
            out = out + expert(h, w[p + "shared.up"], w[p + "shared.down"])
        return out

    def token(self, st, tok, taps=None):
        """One token through every layer; returns its logits.  taps (list) receives the stream after every layer."""
        t = st["n"]
        x = self.w["embed"][tok].copy()
        shared = {}
        for i, L in enumerate(self.cfg["layers"]):
            mix = self.mixer_a if L["type"] == "attention" else self.mixer_b
            x = offset_norm(self.alpha * x + mix(i, x, t, st["layers"][i], shared), self.w["l%d.norm1" % i], self.eps)
            if L.get("mlp") is not None:
                x = offset_norm(self.alpha * x + self.feed_forward(i, x), self.w["l%d.norm2" % i], self.eps)
            if taps is not None:
                taps.append(x.copy())
        st["n"] += 1
        return self.w["head"] @ offset_norm(x, self.w["final.norm"], self.eps)

    def step(self, st, tokens):
        return np.stack([self.token(st, t) for t in tokens])

    def forward(self, tokens, taps=None):
        """Logits of every position [n, vocab]; taps (list) receives [layers][n, width]."""
        st = self.new_state()
        rows, per_tok = [], []
        for t in tokens:
            tp = []
            rows.append(self.token(st, t, tp))
            per_tok.append(tp)
        if taps is not None:
            for i in range(len(self.cfg["layers"])):
                taps.append(np.stack([tp[i] for tp in per_tok]))
        return np.stack(rows)
