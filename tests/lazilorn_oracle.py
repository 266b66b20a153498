"""Plain, slow restatement of the Lazilorn design in numpy (float64 by default), one function per mechanism.

It shares no code with the library: token by token for the recurrent parts, a dense mask for attention.  `Model.forward` runs whole
sequences from position 0; `Model.step` carries an explicit state so that decoding can be compared with it too.

Notation: x is the residual stream [T, width]; W matrices are [out, in]; h is a sublayer's normed input.
"""
import math

import numpy as np


def rms_norm(x, w, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def logsigmoid(z):
    return -np.logaddexp(0.0, -z)


def sinusoid(positions, width):
    """[len(positions), width]: entry 2i = sin(p * 10000^(-2i/width)), entry 2i+1 = cos of the same angle."""
    out = np.zeros((len(positions), width))
    p = np.asarray(positions, dtype=np.float64)[:, None]
    i = np.arange((width + 1) // 2, dtype=np.float64)[None, :]
    ang = p * np.power(10000.0, -2.0 * i / width)
    out[:, 0::2] = np.sin(ang)[:, : out[:, 0::2].shape[1]]
    out[:, 1::2] = np.cos(ang)[:, : out[:, 1::2].shape[1]]
    return out


def visible(i, j, size, keep_first):
    """Sliding window with kept first tokens: may query position i see key position j?"""
    return j <= i and (i - j < size or j < keep_first)


def windowed_attention(q, k, v, q_pos, k_pos, scale, size, keep_first):
    """q [Tq, H, dim], k [Tk, G, dim], v [Tk, G, vdim] -> [Tq, H, vdim]; ordinary softmax over the visible keys."""
    Tq, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((Tq, H, v.shape[2]))
    for a in range(Tq):
        js = [b for b in range(k.shape[0]) if visible(q_pos[a], k_pos[b], size, keep_first)]
        for h in range(H):
            g = h * G // H                     # = floor(h / (H / G))
            s = np.array([q[a, h] @ k[b, g] for b in js]) * scale
            p = np.exp(s - s.max())
            p /= p.sum()
            out[a, h] = sum(p[n] * v[b, g] for n, b in enumerate(js))
    return out


def mlstm_step(state, q, k, v, i_log, f_log):
    """One token of one head of the matrix memory.  state = (S [dim, vdim], n [dim], m scalar); q is already scaled."""
    S, n, m = state
    m_new = max(f_log + m, i_log)
    a = math.exp(f_log + m - m_new)
    b = math.exp(i_log - m_new)
    S = a * S + b * np.outer(k, v)
    n = a * n + b * k
    o = (S.T @ q) / (max(abs(float(n @ q)), math.exp(-m_new)) + 1e-6)
    return (S, n, m_new), o


def delta_step(S, q, k, v, beta, g):
    """One token of one head of the gated delta rule; S [dim, vdim].  The read-out sees this token's write."""
    S = g * S
    u = beta * (v - S.T @ k)
    S = S + np.outer(k, u)
    return S, S.T @ q


def causal_conv_silu(x, w, tail):
    """x [T, C] new inputs, w [C, taps] (last column = current token), tail [taps-1, C] earlier inputs -> (y [T, C], new tail)."""
    taps = w.shape[1]
    full = np.concatenate([tail, x], axis=0)
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        win = full[t : t + taps]                      # inputs t-taps+1 .. t
        y[t] = np.sum(win * w.T, axis=0)
    return silu(y), full[full.shape[0] - (taps - 1):] if taps > 1 else full[:0]


def relu2_mlp(h, up, down):
    return np.square(np.maximum(h @ up.T, 0.0)) @ down.T


class Model:
    """cfg: the parsed config.json (dict); w: name -> float64 array."""

    def __init__(self, cfg, weights, dtype=np.float64):
        self.cfg = cfg
        self.w = {k: np.asarray(v, dtype=dtype) for k, v in weights.items()}
        self.eps = cfg["norm"]["eps"]
        self.width = cfg["width"]
        n = len(cfg["layers"])
        lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
        self.loop = lp
        runs = list(range(0, lp["start"]))
        for _ in range(lp["times"] if lp["stop"] > lp["start"] else 0):
            runs += list(range(lp["start"], lp["stop"]))
        runs += list(range(max(lp["stop"], lp["start"]), n))
        self.runs = runs                 # layer index of every layer run, in order

    # ---- state --------------------------------------------------------------------------------------------------------
    def new_state(self):
        st = {"pos": 0, "runs": []}
        for li in self.runs:
            L = self.cfg["layers"][li]
            m = L["mixer"]
            if L["type"] == "parallel":
                le, ri = m["left"], m["right"]
                st["runs"].append({
                    "k": np.zeros((0, le["kv_heads"], le["dim"])), "v": np.zeros((0, le["kv_heads"], le["vdim"])),
                    "S": np.zeros((ri["heads"], ri["dim"], ri["vdim"])), "n": np.zeros((ri["heads"], ri["dim"])),
                    "m": np.zeros(ri["heads"])})
            else:
                kv, H = m["kv_heads"], m["heads"]
                st["runs"].append({
                    "S": np.zeros((H, m["dim"], m["vdim"])),
                    "cq": np.zeros((m["conv"] - 1, kv * m["dim"])), "ck": np.zeros((m["conv"] - 1, kv * m["dim"])),
                    "cv": np.zeros((m["conv"] - 1, H * m["vdim"]))})
        return st

    # ---- mixers -------------------------------------------------------------------------------------------------------
    def parallel(self, p, m, h, pos, rs):
        w = self.w
        le, ri = m["left"], m["right"]
        T = h.shape[0]
        # left: windowed softmax attention, q/k norm, no rotation, sigmoid output gate
        H, G, d, dv = le["heads"], le["kv_heads"], le["dim"], le["vdim"]
        q = rms_norm((h @ w[p + "left.q"].T).reshape(T, H, d), w[p + "left.q.norm"], self.eps)
        k = rms_norm((h @ w[p + "left.k"].T).reshape(T, G, d), w[p + "left.k.norm"], self.eps)
        v = (h @ w[p + "left.v"].T).reshape(T, G, dv)
        rs["k"] = np.concatenate([rs["k"], k], axis=0)
        rs["v"] = np.concatenate([rs["v"], v], axis=0)
        att = windowed_attention(q, rs["k"], rs["v"], pos, np.arange(rs["k"].shape[0]), le["scale"],
                                 le["mask"]["size"], le["mask"]["keep_first"])
        left = (att.reshape(T, H * dv) * sigmoid(h @ w[p + "left.g"].T)) @ w[p + "left.o"].T
        # right: matrix memory
        H, d, dv, cap = ri["heads"], ri["dim"], ri["vdim"], ri["gate_cap"]
        q = (h @ w[p + "right.q"].T).reshape(T, H, d) * d ** -0.5
        k = (h @ w[p + "right.k"].T).reshape(T, H, d)
        v = (h @ w[p + "right.v"].T).reshape(T, H, dv)
        ig = cap * np.tanh((h @ w[p + "right.i"].T + w[p + "right.i.b"]) / cap)
        fg = logsigmoid(cap * np.tanh((h @ w[p + "right.f"].T + w[p + "right.f.b"]) / cap))
        o = np.zeros((T, H, dv))
        for hh in range(H):
            st = (rs["S"][hh], rs["n"][hh], float(rs["m"][hh]))
            for t in range(T):
                st, o[t, hh] = mlstm_step(st, q[t, hh], k[t, hh], v[t, hh], float(ig[t, hh]), float(fg[t, hh]))
            rs["S"][hh], rs["n"][hh], rs["m"][hh] = st
        o = unit_rms(o, self.eps).reshape(T, H * dv) * w[p + "right.norm"] * sigmoid(h @ w[p + "right.g"].T)
        right = o @ w[p + "right.o"].T
        return m["left_scale"] * left + m["right_scale"] * right

    def delta(self, p, m, h, rs):
        w = self.w
        T = h.shape[0]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        q, rs["cq"] = causal_conv_silu(h @ w[p + "q"].T, w[p + "q.conv"], rs["cq"])
        k, rs["ck"] = causal_conv_silu(h @ w[p + "k"].T, w[p + "k.conv"], rs["ck"])
        v, rs["cv"] = causal_conv_silu(h @ w[p + "v"].T, w[p + "v.conv"], rs["cv"])
        q = q.reshape(T, G, d)
        k = k.reshape(T, G, d)
        v = v.reshape(T, H, dv)
        q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * d ** -0.5
        k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
        beta = sigmoid(h @ w[p + "b"].T)
        g = np.exp(-np.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
        o = np.zeros((T, H, dv))
        for hh in range(H):
            gg = hh * G // H
            S = rs["S"][hh]
            for t in range(T):
                S, o[t, hh] = delta_step(S, q[t, gg], k[t, gg], v[t, hh], beta[t, hh], g[t, hh])
            rs["S"][hh] = S
        o = unit_rms(o, self.eps) * w[p + "norm"]
        o = o.reshape(T, H * dv) * silu(h @ w[p + "g"].T)
        return o @ w[p + "o"].T

    # ---- the model ----------------------------------------------------------------------------------------------------
    def step(self, state, tokens, taps=None):
        """Run `tokens` from `state` (changed in place); returns logits [T, vocab].  taps: list that receives the residual stream
        after every layer run."""
        cfg, w = self.cfg, self.w
        T = len(tokens)
        pos = np.arange(state["pos"], state["pos"] + T)
        x = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"] + sinusoid(pos, self.width)
        lp = self.loop
        looped = lp["stop"] > lp["start"]
        for r, li in enumerate(self.runs):
            if looped and li == lp["start"] and lp["start"] <= li < lp["stop"]:
                t = sum(1 for rr in range(r) if self.runs[rr] == lp["start"])
                x = x + w["loop.step"][t]
            L = cfg["layers"][li]
            p = "l%d." % li
            h = rms_norm(x, w[p + "norm1"], self.eps)
            if L["type"] == "parallel":
                x = x + self.parallel(p + "mix.", L["mixer"], h, pos, state["runs"][r])
            elif L["type"] == "delta":
                x = x + self.delta(p + "mix.", L["mixer"], h, state["runs"][r])
            else:
                raise ValueError(L["type"])
            if L.get("mlp"):
                if L["mlp"]["kind"] != "dense":
                    raise ValueError(L["mlp"]["kind"])
                x = x + relu2_mlp(rms_norm(x, w[p + "norm2"], self.eps), w[p + "mlp.up"], w[p + "mlp.down"])
            if taps is not None:
                taps.append(x.copy())
        state["pos"] += T
        return rms_norm(x, w["final.norm"], self.eps) @ w["head"].T * cfg["logit_scale"]

    def forward(self, tokens, taps=None):
        return self.step(self.new_state(), tokens, taps)
