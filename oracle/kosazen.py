"""Plain numpy (float64) statement of the Kosazen architecture, one function per mechanism — the yardstick the GPU
kernels and the engine are tested against.  It shares no code with the product path: no paging, no folding of the key
projection into the query, no grouping of tokens by expert; attention walks an explicit per-sequence list of cached rows.

Notation: W x for a weight stored [out, in]; positions start at 0 in every sequence.
  block:   x <- x + dyt_1b(mix(dyt_1(x)));   x <- x + dyt_2b(ff(dyt_2(x)))          (ff may be absent)
  dyt:     tanh(alpha * x) * w + b
  mix:     q = Wq h  -> per head [nope | rope];  [c_raw | kr_raw] = Wdkv h;  c = rms(c_raw) * g;  kr = rot(kr_raw)
           k_h = Uk_h c,  v_h = Uv_h c;  score = (q_nope . k_h + rot(q_rope) . kr) * scale;  causal softmax;  Wo concat_h(p v_h)
  ff:      s = softmax(Wr h);  pick the `top` largest s + bias;  w = s[picked] / (sum + 1e-20) * router_scale
           experts e < E: Wd (g * sigmoid(1.702 g) * (u + 1)), g = min(Wg h, lim), u = clip(Wu h, -lim, lim);  e >= E: h itself
           plus a shared expert of the same form for every token
"""
import numpy as np


def bf16_round(a):
    """Nearest-even rounding of float values to bfloat16, returned as float64."""
    u = np.asarray(a, np.float32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32).astype(np.float64)


def random_config(rng, vocab=96, width=40, n_layers=3, loop=None, mlp_mask=None, **over):
    """A small configuration in the checkpoint's config.json form.  `over` overrides mixer / router fields for all layers."""
    layers = []
    for i in range(n_layers):
        mixer = {"heads": over.get("heads", 3), "dim": over.get("dim", 12), "rot_dim": over.get("rot_dim", 6),
                 "vdim": over.get("vdim", 10), "kv_rank": over.get("kv_rank", 20), "scale": over.get("scale", 0.19)}
        mixer["rot"] = {"base": over.get("rot_base", 5000.0), "dims": mixer["rot_dim"]}
        mlp = None
        if mlp_mask is None or mlp_mask[i]:
            mlp = {"kind": "moe", "expert": {"ff": over.get("ff", 24), "limit": over.get("limit", 1.25)},
                   "router": {"experts": over.get("experts", 5), "identity": over.get("identity", 2), "top": over.get("top", 3),
                              "scale": over.get("router_scale", 1.3)}}
            if over.get("shared", True):
                mlp["shared"] = {"ff": over.get("shared_ff", 28), "limit": over.get("shared_limit", 0.9)}
        layers.append({"type": "latent_attention", "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Kosazen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": layers}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def tensor_shapes(cfg):
    W, out = cfg["width"], {}
    def norm(name):
        out[name], out[name + ".b"], out[name + ".alpha"] = (W,), (W,), ()
    out["embed"] = (cfg["vocab"], W)
    for i, l in enumerate(cfg["layers"]):
        p, m = "l%d." % i, l["mixer"]
        norm(p + "norm1"); norm(p + "norm1b")
        out[p + "mix.q"] = (m["heads"] * (m["dim"] + m["rot_dim"]), W)
        out[p + "mix.dkv"] = (m["kv_rank"] + m["rot_dim"], W)
        out[p + "mix.dkv.norm"] = (m["kv_rank"],)
        out[p + "mix.uk"] = (m["heads"] * m["dim"], m["kv_rank"])
        out[p + "mix.uv"] = (m["heads"] * m["vdim"], m["kv_rank"])
        out[p + "mix.o"] = (W, m["heads"] * m["vdim"])
        f = l["mlp"]
        if f is not None:
            norm(p + "norm2"); norm(p + "norm2b")
            r = f["router"]
            for e in range(r["experts"]):
                out[p + "mlp.e%d.gate" % e] = (f["expert"]["ff"], W)
                out[p + "mlp.e%d.up" % e] = (f["expert"]["ff"], W)
                out[p + "mlp.e%d.down" % e] = (W, f["expert"]["ff"])
            out[p + "mlp.router"] = (r["experts"] + r.get("identity", 0), W)
            out[p + "mlp.correction"] = (r["experts"] + r.get("identity", 0),)
            if f.get("shared"):
                out[p + "mlp.shared.gate"] = (f["shared"]["ff"], W)
                out[p + "mlp.shared.up"] = (f["shared"]["ff"], W)
                out[p + "mlp.shared.down"] = (W, f["shared"]["ff"])
    norm("final.norm")
    out["head"] = (cfg["vocab"], W)
    return out


def random_weights(cfg, rng, std=None):
    """bf16-representable random tensors {name: float64 array}: matrices ~ N(0, 1/fan_in), norm weights and alphas near 1."""
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(".alpha"):
            v = np.asarray(1.0 + 0.2 * rng.standard_normal())
        elif "norm" in name and not name.endswith(".b"):
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif name.endswith(".b") or name.endswith("correction"):
            v = 0.1 * rng.standard_normal(shape)
        elif name == "embed":
            v = rng.standard_normal(shape)
        else:
            v = rng.standard_normal(shape) * (std if std is not None else 1.0 / np.sqrt(shape[-1]))
        w[name] = bf16_round(v).reshape(shape)
    return w


def to_bf16_bits(a):
    return (np.asarray(a, np.float32).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def layer_runs(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


# ------------------------------------------------------------------------------------------------ mechanisms


def dyt(x, w, name):
    return np.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def rms_norm(x, g, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * g


def rotate_pairs(x, pos, dims, base):
    """Interleaved rotary: (x[2i], x[2i+1]) turned by pos * base^(-2i/dims) for the first `dims` entries of the last axis."""
    x = np.array(x, np.float64)
    for i in range(dims // 2):
        a = pos * base ** (-2.0 * i / dims)
        u, v = x[..., 2 * i].copy(), x[..., 2 * i + 1].copy()
        x[..., 2 * i] = u * np.cos(a) - v * np.sin(a)
        x[..., 2 * i + 1] = v * np.cos(a) + u * np.sin(a)
    return x


def latent_rows(h, w, p, m, eps, pos):
    """What one token leaves in the cache: (normed latent, rotated shared key part)."""
    dkv = w[p + "dkv"] @ h
    r = m["kv_rank"]
    return rms_norm(dkv[:r], w[p + "dkv.norm"], eps), rotate_pairs(dkv[r:], pos, m["rot"]["dims"], m["rot"]["base"])


def latent_attention_token(h, w, p, m, pos, cached):
    """Output of the mixer for one token at `pos`, given the cached rows [(c_j, kr_j)] of positions 0..pos (own row last)."""
    H, d, rd, vd = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = (w[p + "q"] @ h).reshape(H, d + rd)
    out = np.zeros(H * vd)
    for hh in range(H):
        qn, qr = q[hh, :d], rotate_pairs(q[hh, d:], pos, m["rot"]["dims"], m["rot"]["base"])
        uk, uv = w[p + "uk"][hh * d:(hh + 1) * d], w[p + "uv"][hh * vd:(hh + 1) * vd]
        s = np.array([(qn @ (uk @ c) + qr @ kr) * m["scale"] for c, kr in cached])
        e = np.exp(s - s.max())
        pr = e / e.sum()
        out[hh * vd:(hh + 1) * vd] = sum(pj * (uv @ c) for pj, (c, _) in zip(pr, cached))
    return w[p + "o"] @ out


def glu_expert(h, wg, wu, wd, limit):
    g = np.minimum(wg @ h, limit)
    u = np.clip(wu @ h, -limit, limit)
    return wd @ (g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0))


def route(h, w, p, r):
    """(indices, weights, margin): margin = gap between the last chosen and the best rejected selection score."""
    z = w[p + "router"] @ h
    e = np.exp(z - z.max())
    s = e / e.sum()
    sel = s + w[p + "correction"]
    order = np.argsort(-sel, kind="stable")
    idx = order[:r["top"]]
    wt = s[idx] / (s[idx].sum() + 1e-20) * r["scale"]
    margin = sel[order[r["top"] - 1]] - sel[order[r["top"]]] if len(order) > r["top"] else np.inf
    return idx, wt, margin


def moe(h, w, p, f, margins=None):
    r = f["router"]
    idx, wt, margin = route(h, w, p, r)
    if margins is not None:
        margins.append(margin)
    out = np.zeros_like(h)
    for e, we in zip(idx, wt):
        if e < r["experts"]:
            q = p + "e%d." % e
            out += we * glu_expert(h, w[q + "gate"], w[q + "up"], w[q + "down"], f["expert"]["limit"])
        else:
            out += we * h
    if f.get("shared"):
        q = p + "shared."
        out += glu_expert(h, w[q + "gate"], w[q + "up"], w[q + "down"], f["shared"]["limit"])
    return out


# ------------------------------------------------------------------------------------------------ model


class Sequence:
    """One request's state: per layer run the list of cached (latent, key part) rows."""

    def __init__(self, cfg):
        self.cache = [[] for _ in layer_runs(cfg)]
        self.n = 0


def step_token(cfg, w, seq, token, residuals=None, margins=None):
    """Feeds ONE token to a sequence; returns its logits.  residuals (list): gets the residual stream after every layer run;
    margins (list): gets every router's gap between the last chosen and the best rejected selection score."""
    eps = cfg["norm"]["eps"]
    x = np.array(w["embed"][token], np.float64)
    pos = seq.n
    for r, li in enumerate(layer_runs(cfg)):
        l, p = cfg["layers"][li], "l%d." % li
        h = dyt(x, w, p + "norm1")
        seq.cache[r].append(latent_rows(h, w, p + "mix.", l["mixer"], eps, pos))
        x = x + dyt(latent_attention_token(h, w, p + "mix.", l["mixer"], pos, seq.cache[r]), w, p + "norm1b")
        if l["mlp"] is not None:
            x = x + dyt(moe(dyt(x, w, p + "norm2"), w, p + "mlp.", l["mlp"], margins), w, p + "norm2b")
        if residuals is not None:
            residuals.append(x.copy())
    seq.n += 1
    return w["head"] @ dyt(x, w, "final.norm")


def logits_of(cfg, w, tokens, router_margins=None):
    """[len(tokens), vocab] logits of a whole sequence, token by token.  router_margins (list): gets, per position, the
    smallest router margin on its way through the layers (a reduced-precision run may choose differently where it is tiny)."""
    s = Sequence(cfg)
    out = []
    for t in tokens:
        m = []
        out.append(step_token(cfg, w, s, t, margins=m))
        if router_margins is not None:
            router_margins.append(min(m) if m else np.inf)
    return np.stack(out)


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
