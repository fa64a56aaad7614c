"""Plain numpy (float64) statement of the Talapel architecture, one function per mechanism: the yardstick the GPU kernels
and the engine are tested against.  It shares no code with the product path: no paging, no state slots, no packing of
projections, no grouping of tokens by expert.  Every sequence is walked token by token; attention keeps an explicit list of
key / value rows, the recurrent mixers keep their state matrices as arrays.

Notation: W x for a weight stored [out, in]; positions start at 0 in every sequence; rms(v) = v / sqrt(mean(v^2) + eps).
  layer:      h = ln(x) * w;  x <- x + mixer(h) + ff(h)                         (one norm, both branches read it; ff may be absent)
  ln:         (x - mean) / sqrt(var + eps), var = mean of squared deviations
  loop:       layers start..stop-1 run `times` times on the same weights; every pass begins with x <- W_loop [x ; x0],
              x0 = the scaled embedding; every layer run has its own cache / state
  parallel:   c_l * attention(h) + c_r * ssd(h)
  attention:  q, k, v with biases; grouped heads; q *= 1 + coef * ln(floor((p + 1) / every) + 1); s = cap * tanh(q.k * scale / cap);
              causal softmax; concat * sigmoid(Wg h); Wo (+ bias)
  ssd:        [z | x | B | C | dt] = W_in h;  (x, B, C) <- silu(causal conv over the last `taps` tokens + bias);
              dt <- softplus(dt + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x;
              Wo (rms_groups(y * silu(z)) * w)
  retention:  q, k rotated (rotate-half pairing on the first rot dims), k *= dim^-1/2;  S <- decay_h S + k v^T;  o = S^T q;
              Wo (concat_h rms(o_h) * silu(Wg h))
  ff dense:   Wd (silu(Wg h) * (Wu h))
  ff experts: a table row per token id names `top` experts, each weighted 1/top;  expert: Wd relu(Wu h)^2
"""
import numpy as np


def bf16_round(a):
    """Nearest-even rounding of float values to bfloat16, returned as float64."""
    u = np.asarray(a, np.float32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32).astype(np.float64)


def to_bf16_bits(a):
    """bf16-representable float values -> uint16 bit patterns (integer arrays pass as int32)."""
    a = np.asarray(a)
    if a.dtype.kind in "iu":
        return a.astype(np.int32)
    return (np.ascontiguousarray(a, np.float32).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


# ---- configuration / weights --------------------------------------------------------------------------------------------
def parallel_mixer(heads=4, kv_heads=2, dim=6, vdim=10, scale=0.3, softcap=8.0, coef=0.4, every=3, s_heads=3, groups=1,
                   state=5, s_vdim=4, taps=3, norm_groups=1, left_scale=0.9, right_scale=1.3):
    return {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
                     "q_temp": {"coef": coef, "every": every}},
            "right": {"heads": s_heads, "groups": groups, "state": state, "vdim": s_vdim, "conv": taps, "norm_groups": norm_groups},
            "left_scale": left_scale, "right_scale": right_scale}


def retention_mixer(heads=3, dim=8, vdim=6, rot_dims=4, rot_base=100.0, decay=None):
    if decay is None:
        decay = [1.0 - 2.0 ** (-2 - i) for i in range(heads)]
    return {"heads": heads, "dim": dim, "vdim": vdim, "rot": {"base": rot_base, "dims": rot_dims}, "decay": list(decay)}


def dense_mlp(ff=24):
    return {"kind": "dense", "ff": ff}


def expert_mlp(experts=5, top=2, ff=12):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def make_config(layers, vocab=80, width=24, loop=None, eps=1e-5, embed_scale=3.0):
    """layers: list of (type, mixer dict, mlp dict or None)."""
    cfg = {"architecture": "Talapel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
           "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers]}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def has_loop(cfg):
    return isinstance(cfg.get("loop"), dict)


def tensor_shapes(cfg):
    W, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], W)
    if has_loop(cfg):
        out["loop.in"] = (W, 2 * W)
    for i, l in enumerate(cfg["layers"]):
        p, m = "l%d." % i, l["mixer"]
        out[p + "norm1"] = (W,)
        if l["type"] == "parallel":
            a, s = m["left"], m["right"]
            q = p + "mix.left."
            out[q + "q"], out[q + "q.b"] = (a["heads"] * a["dim"], W), (a["heads"] * a["dim"],)
            out[q + "k"], out[q + "k.b"] = (a["kv_heads"] * a["dim"], W), (a["kv_heads"] * a["dim"],)
            out[q + "v"], out[q + "v.b"] = (a["kv_heads"] * a["vdim"], W), (a["kv_heads"] * a["vdim"],)
            out[q + "g"] = (a["heads"] * a["vdim"], W)
            out[q + "o"], out[q + "o.b"] = (W, a["heads"] * a["vdim"]), (W,)
            r = p + "mix.right."
            inner, gn = s["heads"] * s["vdim"], s["groups"] * s["state"]
            out[r + "in"] = (2 * inner + 2 * gn + s["heads"], W)
            out[r + "conv"], out[r + "conv.b"] = (inner + 2 * gn, s["conv"]), (inner + 2 * gn,)
            out[r + "dt_bias"] = out[r + "A_log"] = out[r + "D"] = (s["heads"],)
            out[r + "norm"] = (inner,)
            out[r + "o"] = (W, inner)
        else:
            q = p + "mix."
            out[q + "q"] = out[q + "k"] = (m["heads"] * m["dim"], W)
            out[q + "v"] = out[q + "g"] = (m["heads"] * m["vdim"], W)
            out[q + "o"] = (W, m["heads"] * m["vdim"])
        f = l["mlp"]
        if f is None:
            continue
        if f["kind"] == "dense":
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (f["ff"], W)
            out[p + "mlp.down"] = (W, f["ff"])
        else:
            for e in range(f["router"]["experts"]):
                out[p + "mlp.e%d.up" % e] = (f["expert"]["ff"], W)
                out[p + "mlp.e%d.down" % e] = (W, f["expert"]["ff"])
            out[p + "mlp.table"] = (cfg["vocab"], f["router"]["top"])
    out["final.norm"] = (W,)
    out["head"] = (cfg["vocab"], W)
    return out


def random_weights(cfg, rng, std=None):
    """bf16-representable float64 weights; expert tables are int32 with distinct entries per row."""
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last == "table":
            e = cfg["layers"][int(name[1:name.index(".")])]["mlp"]["router"]["experts"]
            w[name] = np.stack([rng.permutation(e)[:shape[1]] for _ in range(shape[0])]).astype(np.int32)
            continue
        if "norm" in name:
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "A_log":
            a = rng.uniform(-1.5, 0.5, shape)
        elif last == "dt_bias":
            a = rng.uniform(-2.0, 0.5, shape)
        elif last == "D":
            a = rng.uniform(0.5, 1.5, shape)
        elif last == "b":
            a = 0.3 * rng.standard_normal(shape)
        elif last == "conv":
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
        else:
            s = std if std is not None else 1.0 / np.sqrt(shape[-1])
            a = s * rng.standard_normal(shape)
        w[name] = bf16_round(a)
    return w


def layer_runs(cfg):
    """[(layer index, first of its pass?)] in execution order."""
    n = len(cfg["layers"])
    if not has_loop(cfg):
        return [(i, False) for i in range(n)]
    lp = cfg["loop"]
    runs = [(i, False) for i in range(lp["start"])]
    for _ in range(lp["times"]):
        runs += [(i, i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, False) for i in range(lp["stop"], n)]


# ---- mechanisms ---------------------------------------------------------------------------------------------------------
def layer_norm(x, weight, eps):
    d = x - x.mean()
    return d / np.sqrt((d * d).mean() + eps) * weight


def rms(x, eps):
    return x / np.sqrt((x * x).mean() + eps)


def silu(x):
    return x / (1.0 + np.exp(-x))


def softplus(x):
    return np.logaddexp(0.0, x)


def query_temperature(pos, coef, every):
    return 1.0 + coef * np.log(np.floor((pos + 1) / every) + 1.0)


def capped_attention_token(h, w, p, m, pos, rows):
    """Softmax attention of one token.  rows: this sequence's (k, v) list for this layer run; the token's own pair is appended."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (w[p + "q"] @ h + w[p + "q.b"]).reshape(H, D) * query_temperature(pos, m["q_temp"]["coef"], m["q_temp"]["every"])
    rows.append(((w[p + "k"] @ h + w[p + "k.b"]).reshape(G, D), (w[p + "v"] @ h + w[p + "v.b"]).reshape(G, V)))
    out = np.zeros((H, V))
    for hh in range(H):
        g = hh // (H // G)
        s = np.array([q[hh] @ k[g] for k, _ in rows]) * m["scale"]
        if m.get("softcap", 0.0) > 0.0:
            s = m["softcap"] * np.tanh(s / m["softcap"])
        e = np.exp(s - s.max())
        e /= e.sum()
        out[hh] = sum(pj * v[g] for pj, (_, v) in zip(e, rows))
    gate = 1.0 / (1.0 + np.exp(-(w[p + "g"] @ h)))
    return w[p + "o"] @ (out.reshape(-1) * gate) + w[p + "o.b"]


class SsdState:
    def __init__(self, m):
        ch = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
        self.window = np.zeros((m["conv"] - 1, ch))          # the raw inputs of the last taps - 1 tokens, oldest first
        self.S = np.zeros((m["heads"], m["state"], m["vdim"]))


def ssd_token(h, w, p, m, eps, st):
    """State-space-duality mixer of one token; st (SsdState) is advanced."""
    Hh, G, N, P, K = m["heads"], m["groups"], m["state"], m["vdim"], m["conv"]
    inner = Hh * P
    u = w[p + "in"] @ h
    z, xbc, dt = u[:inner], u[inner:2 * inner + 2 * G * N], u[2 * inner + 2 * G * N:]
    win = np.vstack([st.window, xbc[None]])                  # [taps, channels], the last row is this token's
    st.window = win[1:]
    xbc = silu((win * w[p + "conv"].T).sum(0) + w[p + "conv.b"])
    x, B, C = xbc[:inner].reshape(Hh, P), xbc[inner:inner + G * N].reshape(G, N), xbc[inner + G * N:].reshape(G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    y = np.zeros((Hh, P))
    for hh in range(Hh):
        g = hh // (Hh // G)
        st.S[hh] = np.exp(-np.exp(w[p + "A_log"][hh]) * dt[hh]) * st.S[hh] + dt[hh] * np.outer(B[g], x[hh])
        y[hh] = st.S[hh].T @ C[g] + w[p + "D"][hh] * x[hh]
    t = y.reshape(-1) * silu(z)
    t = np.concatenate([rms(part, eps) for part in np.split(t, m["norm_groups"])]) * w[p + "norm"]
    return w[p + "o"] @ t


def rotate_half(v, pos, dims, base):
    """Rotary position on the first `dims` values of every row of v (rows = heads): dimension i pairs with i + dims/2."""
    out = v.copy()
    half = dims // 2
    if half == 0:
        return out
    ang = pos * base ** (-2.0 * np.arange(half) / dims)
    a, b = v[:, :half], v[:, half:dims]
    out[:, :half] = a * np.cos(ang) - b * np.sin(ang)
    out[:, half:dims] = b * np.cos(ang) + a * np.sin(ang)
    return out


def retention_token(h, w, p, m, eps, pos, S):
    """Decayed linear attention of one token; S [heads, dim, vdim] is advanced in place."""
    Hh, D, V = m["heads"], m["dim"], m["vdim"]
    q = rotate_half((w[p + "q"] @ h).reshape(Hh, D), pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half((w[p + "k"] @ h).reshape(Hh, D), pos, m["rot"]["dims"], m["rot"]["base"]) * D ** -0.5
    v = (w[p + "v"] @ h).reshape(Hh, V)
    o = np.zeros((Hh, V))
    for hh in range(Hh):
        S[hh] = m["decay"][hh] * S[hh] + np.outer(k[hh], v[hh])
        o[hh] = rms(S[hh].T @ q[hh], eps)
    return w[p + "o"] @ (o.reshape(-1) * silu(w[p + "g"] @ h))


def dense_ff(h, w, p):
    return w[p + "down"] @ (silu(w[p + "gate"] @ h) * (w[p + "up"] @ h))


def table_experts(h, w, p, f, token):
    out = 0.0
    for e in w[p + "table"][token]:
        out = out + w[p + "e%d.down" % e] @ np.maximum(w[p + "e%d.up" % e] @ h, 0.0) ** 2
    return out / f["router"]["top"]


# ---- model --------------------------------------------------------------------------------------------------------------
class Sequence:
    """Everything one sequence carries from token to token: per layer run its attention rows and recurrent states."""

    def __init__(self, cfg):
        self.n = 0
        self.state = []
        for li, _ in layer_runs(cfg):
            l = cfg["layers"][li]
            if l["type"] == "parallel":
                self.state.append(([], SsdState(l["mixer"]["right"])))
            else:
                m = l["mixer"]
                self.state.append(np.zeros((m["heads"], m["dim"], m["vdim"])))


def step_token(cfg, w, seq, token, residuals=None):
    """Runs one token of sequence `seq`; returns its logits.  residuals (list): gets the stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x0 = np.array(w["embed"][token], np.float64) * cfg["embedding"]["scale"]
    x, pos = x0.copy(), seq.n
    for r, (li, first) in enumerate(layer_runs(cfg)):
        l, p = cfg["layers"][li], "l%d." % li
        if first:
            x = w["loop.in"] @ np.concatenate([x, x0])
        h = layer_norm(x, w[p + "norm1"], eps)
        if l["type"] == "parallel":
            m = l["mixer"]
            rows, st = seq.state[r]
            mix = m["left_scale"] * capped_attention_token(h, w, p + "mix.left.", m["left"], pos, rows) + \
                m["right_scale"] * ssd_token(h, w, p + "mix.right.", m["right"], eps, st)
        else:
            mix = retention_token(h, w, p + "mix.", l["mixer"], eps, pos, seq.state[r])
        f = l["mlp"]
        if f is not None:
            mix = mix + (dense_ff(h, w, p + "mlp.") if f["kind"] == "dense" else table_experts(h, w, p + "mlp.", f, token))
        x = x + mix
        if residuals is not None:
            residuals.append(x.copy())
    seq.n += 1
    return w["head"] @ layer_norm(x, w["final.norm"], eps)


def logits_of(cfg, w, tokens):
    s = Sequence(cfg)
    return np.stack([step_token(cfg, w, s, t) for t in tokens])


def greedy(cfg, w, prompt, n_new):
    """(generated tokens, top-1 / top-2 logit margin of every choice)."""
    s = Sequence(cfg)
    lg = None
    for t in prompt:
        lg = step_token(cfg, w, s, t)
    out, margins = [], []
    for _ in range(n_new):
        o = np.argsort(-lg, kind="stable")
        out.append(int(o[0]))
        margins.append(float(lg[o[0]] - lg[o[1]]))
        lg = step_token(cfg, w, s, out[-1])
    return out, margins
