"""Plain float64 restatement of the Vakesun design, one function per mechanism, for the tests. It shares no code with the engine.

A model is (cfg, weights): cfg is the config.json tree, weights maps tensor names to torch tensors. x [T, W] is the residual stream of T
tokens of one sequence at positions 0 .. T-1; m = cfg["residual_mult"].

  embedding:   x = embed[token] * embedding.scale
  layer:       x <- x + m * dyt_1b(mixer(dyt_1(x)));  x <- x + m * dyt_2b(ff(dyt_2(x)))  (no second sublayer when "mlp" is null)
               x <- x + m * unit_rms(Wp (gelu_tanh(Wg x) * e)) * side.norm,  e = side.embed[token, layer * sd : (layer + 1) * sd]
  dyt:         tanh(alpha * x) * w + b      (no mean, no variance)
  attention:   q, k = rotate_p(unit_rms(W h per head) * weight) over the first rot.dims channels, pair (i, i + dims/2), YaRN-blended
               frequencies; softmax_j<=i(scale * q_i . k_j); grouped key / value heads; Wo
  mlstm:       i = cap tanh((Wi h + bi) / cap), f = logsigmoid(cap tanh((Wf h + bf) / cap)); m_t = max(f + m_(t-1), i) with m_0 = 0;
               S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T, n_t likewise with k; o = S_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6),
               q = Wq h / sqrt(dim); Wo (unit_rms(o per head) * norm * sigmoid(Wg h))
  latent:      cq = unit_rms(Wdq h) * wq, q = Wuq cq; c = unit_rms(Wdkv h) * wc (or the lender layer's c); k = Wuk c, v = Wuv c;
               key j visible to i when 0 <= i - j < size; softmax whose denominator also holds exp(sink_h); head output times
               sigmoid(Wg h)_h; Wo
  ff:          Wd relu(Wu h)^2
  readout:     embed . dyt_final(x)
"""
import math

import torch

F64 = torch.float64


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def dyt(x, W, name):
    """Dynamic Tanh: tanh(alpha x) w + b with the scalar `name.alpha` and the vectors `name`, `name.b`"""
    return torch.tanh(W[name + ".alpha"].to(F64) * x.to(F64)) * W[name].to(F64) + W[name + ".b"].to(F64)


def rot_frequencies(rot):
    """Frequencies of the dims/2 pairs and the factor on cos / sin (1 without scaling)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_halves(x, positions, rot):
    """x [T, heads, n]: channel i pairs with channel i + dims/2 (i < dims/2); channels from `dims` on pass unchanged."""
    x = x.to(F64)
    dims = int(rot["dims"])
    half = dims // 2
    f, mult = rot_frequencies(rot)
    ang = torch.as_tensor(positions, dtype=F64)[:, None] * torch.tensor(f, dtype=F64)[None, :]       # [T, half]
    c, s = (torch.cos(ang) * mult)[:, None, :], (torch.sin(ang) * mult)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def softmax_attention(q, k, v, pos_q, pos_k, scale, window=0, sink=None):
    """q [Tq, H, d], k [Tk, G, d], v [Tk, G, dv] -> [Tq, H, dv]; the key at pos_k[j] is visible from pos_q[i] when 0 <= i - j (and
    i - j < window, if there is one); query head h reads key / value head h // (H / G). sink [H]: one more term exp(sink_h) in the
    denominator, with no key and no value."""
    Tq, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    kk, vv = k.to(F64).repeat_interleave(H // G, dim=1), v.to(F64).repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->ihj", q.to(F64), kk) * scale
    dist = torch.as_tensor(pos_q)[:, None] - torch.as_tensor(pos_k)[None, :]
    seen = dist >= 0
    if window:
        seen = seen & (dist < window)
    s = s.masked_fill(~seen[:, None, :], -math.inf)
    if sink is not None:
        s = torch.cat([s, sink.to(F64)[None, :, None].expand(Tq, H, 1)], dim=2)
    w = torch.softmax(s, dim=2)
    if sink is not None:
        w = w[..., :-1]
    return torch.einsum("ihj,jhv->ihv", w, vv)


def attention_mixer(h, W, p, mc, eps, positions, past=None):
    """past = (k, v, positions) of earlier tokens, already normed and rotated -> (output [T, width], (k, v, positions) with these tokens)"""
    h = h.to(F64)
    T = h.shape[0]
    H, G, d, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    q = (h @ W[p + "mix.q"].to(F64).T).reshape(T, H, d)
    k = (h @ W[p + "mix.k"].to(F64).T).reshape(T, G, d)
    v = (h @ W[p + "mix.v"].to(F64).T).reshape(T, G, dv)
    q = unit_rms(q, eps) * W[p + "mix.q.norm"].to(F64)
    k = unit_rms(k, eps) * W[p + "mix.k.norm"].to(F64)
    if mc.get("rot"):
        q = rotate_halves(q, positions, mc["rot"])
        k = rotate_halves(k, positions, mc["rot"])
    pos_k = list(positions)
    if past is not None:
        k, v, pos_k = torch.cat([past[0], k]), torch.cat([past[1], v]), list(past[2]) + pos_k
    o = softmax_attention(q, k, v, list(positions), pos_k, float(mc["scale"]))
    return o.reshape(T, H * dv) @ W[p + "mix.o"].to(F64).T, (k, v, pos_k)


def mlstm_gates(i_pre, f_pre, cap):
    """log input gate and log forget gate from the biased projections"""
    i = cap * torch.tanh(i_pre.to(F64) / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh(f_pre.to(F64) / cap))
    return i, f


def mlstm_scan(q, k, v, i, f, state=None):
    """q, k [T, H, d] (q already scaled), v [T, H, dv], i, f [T, H]; state = (S [H, d, dv], n [H, d], m [H]) -> (o [T, H, dv], state)"""
    T, H, d = q.shape
    dv = v.shape[2]
    if state is None:
        state = (torch.zeros(H, d, dv, dtype=F64), torch.zeros(H, d, dtype=F64), torch.zeros(H, dtype=F64))
    S, n, m = (t.to(F64).clone() for t in state)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(f[t] + m, i[t])
        keep, take = torch.exp(f[t] + m - m_new), torch.exp(i[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        o[t] = num / den[:, None]
    return o, (S, n, m)


def mlstm_mixer(h, W, p, mc, eps, state=None):
    h = h.to(F64)
    T = h.shape[0]
    H, d, dv, cap = mc["heads"], mc["dim"], mc["vdim"], float(mc["gate_cap"])
    q = (h @ W[p + "mix.q"].to(F64).T).reshape(T, H, d) * d ** -0.5
    k = (h @ W[p + "mix.k"].to(F64).T).reshape(T, H, d)
    v = (h @ W[p + "mix.v"].to(F64).T).reshape(T, H, dv)
    i, f = mlstm_gates(h @ W[p + "mix.i"].to(F64).T + W[p + "mix.i.b"].to(F64), h @ W[p + "mix.f"].to(F64).T + W[p + "mix.f.b"].to(F64), cap)
    o, state = mlstm_scan(q, k, v, i, f, state)
    o = unit_rms(o, eps).reshape(T, H * dv) * W[p + "mix.norm"].to(F64) * torch.sigmoid(h @ W[p + "mix.g"].to(F64).T)
    return o @ W[p + "mix.o"].to(F64).T, state


def latent_attention_mixer(h, W, p, mc, eps, positions, past=None, lent=None):
    """past = (c, positions) of earlier tokens; lent = the lender layer's (c, positions) INCLUDING these tokens (a layer with kv_from)
    -> (output, (c, positions))"""
    h = h.to(F64)
    T = h.shape[0]
    H, d, dv = mc["heads"], mc["dim"], mc["vdim"]
    cq = unit_rms(h @ W[p + "mix.dq"].to(F64).T, eps) * W[p + "mix.dq.norm"].to(F64)
    q = (cq @ W[p + "mix.uq"].to(F64).T).reshape(T, H, d)
    if lent is not None:
        c, pos_k = lent
    else:
        c = unit_rms(h @ W[p + "mix.dkv"].to(F64).T, eps) * W[p + "mix.dkv.norm"].to(F64)
        pos_k = list(positions)
        if past is not None:
            c, pos_k = torch.cat([past[0], c]), list(past[1]) + pos_k
    k = (c @ W[p + "mix.uk"].to(F64).T).reshape(-1, H, d)
    v = (c @ W[p + "mix.uv"].to(F64).T).reshape(-1, H, dv)
    window = int(mc["mask"]["size"]) if mc.get("mask") else 0
    o = softmax_attention(q, k, v, list(positions), pos_k, float(mc["scale"]), window=window, sink=W[p + "mix.sink"])
    o = o * torch.sigmoid(h @ W[p + "mix.g"].to(F64).T)[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "mix.o"].to(F64).T, (c, pos_k)


def relu2_ff(h, W, p):
    u = torch.relu(h.to(F64) @ W[p + "mlp.up"].to(F64).T)
    return (u * u) @ W[p + "mlp.down"].to(F64).T


def token_side(x, tokens, W, p, layer, sd, eps):
    """the per-layer token input: what is added to the residual stream, before the factor m"""
    e = W["side.embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long), layer * sd:(layer + 1) * sd]
    g = gelu_tanh(x.to(F64) @ W[p + "side.gate"].to(F64).T) * e
    return unit_rms(g @ W[p + "side.proj"].to(F64).T, eps) * W[p + "side.norm"].to(F64)


def new_state(cfg):
    return {"pos": 0, "layers": [None] * len(cfg["layers"])}


def forward(cfg, W, tokens, state=None):
    """tokens of one sequence continuing `state` (None = from the start) -> (logits [T, vocab], residual after every layer [L, T, W], state)"""
    if state is None:
        state = new_state(cfg)
    eps, m = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    sd = int(cfg["token_side"]["dim"]) if cfg.get("token_side") else 0
    T = len(tokens)
    positions = list(range(state["pos"], state["pos"] + T))
    x = W["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    per_layer = []
    for li, lc in enumerate(cfg["layers"]):
        p = "l%d." % li
        mc = lc["mixer"]
        h = dyt(x, W, p + "norm1")
        if lc["type"] == "attention":
            y, state["layers"][li] = attention_mixer(h, W, p, mc, eps, positions, state["layers"][li])
        elif lc["type"] == "mlstm":
            y, state["layers"][li] = mlstm_mixer(h, W, p, mc, eps, state["layers"][li])
        elif lc["type"] == "latent_attention":
            if mc.get("kv_from") is not None:
                y, _ = latent_attention_mixer(h, W, p, mc, eps, positions, lent=state["layers"][mc["kv_from"]])
            else:
                y, state["layers"][li] = latent_attention_mixer(h, W, p, mc, eps, positions, past=state["layers"][li])
        else:
            raise ValueError(lc["type"])
        x = x + m * dyt(y, W, p + "norm1b")
        if lc.get("mlp"):
            x = x + m * dyt(relu2_ff(dyt(x, W, p + "norm2"), W, p), W, p + "norm2b")
        if sd:
            x = x + m * token_side(x, tokens, W, p, li, sd, eps)
        per_layer.append(x.clone())
    state["pos"] += T
    logits = dyt(x, W, "final.norm") @ W["embed"].to(F64).T
    return logits, torch.stack(per_layer), state


# ---- small configurations and random weights for the tests -----------------------------------------------------------------------------
def attention_layer(heads, kv_heads, dim, vdim, mlp_ff=None, rot_dims=None, base=10000.0, scaling=None, scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    rot_dims = dim if rot_dims is None else rot_dims
    if rot_dims:
        mixer["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            mixer["rot"]["scaling"] = scaling
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": mlp_ff} if mlp_ff else None}


def mlstm_layer(heads, dim, vdim, mlp_ff=None, gate_cap=15.0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}, "mlp": {"kind": "dense", "ff": mlp_ff} if mlp_ff else None}


def latent_layer(heads, dim, vdim, kv_rank, q_rank, window, mlp_ff=None, scale=None, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "mask": {"size": window},
             "scale": dim ** -0.5 if scale is None else scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": mlp_ff} if mlp_ff else None}


def make_config(width, vocab, layers, eps=1e-6, residual_mult=0.5, embedding_scale=1.0, side_dim=8):
    return {"architecture": "Vakesun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "residual_mult": residual_mult,
            "embedding": {"scale": embedding_scale}, "token_side": {"dim": side_dim}, "layers": layers}


def random_weights(cfg, seed=0):
    """bf16-exact random tensors (torch.bfloat16) with spreads that keep every mechanism active: gates away from saturation, sinks of the
    size of the scores, norm scalars near 1."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    sd = cfg["token_side"]["dim"] if cfg.get("token_side") else 0
    w = {}

    def mat(rows, cols, gain=1.0):
        return (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vec(n, mean=0.0, spread=0.1):
        return (mean + spread * torch.randn(n, generator=g)).to(torch.bfloat16)

    def norm(name, alpha):
        w[name], w[name + ".b"] = vec(W, 1.0, 0.2), vec(W, 0.0, 0.1)
        w[name + ".alpha"] = torch.tensor(alpha * (1.0 + 0.2 * float(torch.randn((), generator=g)))).to(torch.bfloat16)

    w["embed"] = mat(V, W, math.sqrt(W))
    if sd:
        w["side.embed"] = mat(V, len(cfg["layers"]) * sd, math.sqrt(len(cfg["layers"]) * sd))
    norm("final.norm", 0.6)
    for i, lc in enumerate(cfg["layers"]):
        p, m = "l%d." % i, lc["mixer"]
        norm(p + "norm1", 0.7)
        norm(p + "norm1b", 1.0)
        if lc["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(H * d, W, 1.5), mat(G * d, W, 1.5), mat(G * dv, W)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = vec(d, 1.0, 0.2), vec(d, 1.0, 0.2)
            w[p + "mix.o"] = mat(W, H * dv)
        elif lc["type"] == "mlstm":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.g"] = mat(H * d, W, 1.5), mat(H * d, W, 1.5), mat(H * dv, W), mat(H * dv, W, 1.5)
            w[p + "mix.i"], w[p + "mix.i.b"] = mat(H, W, 2.0), vec(H, 0.0, 1.0)
            w[p + "mix.f"], w[p + "mix.f.b"] = mat(H, W, 2.0), vec(H, 3.0, 1.0)
            w[p + "mix.norm"], w[p + "mix.o"] = vec(H * dv, 1.0, 0.2), mat(W, H * dv)
        else:
            H, d, dv, R, Q = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            w[p + "mix.dq"], w[p + "mix.dq.norm"], w[p + "mix.uq"] = mat(Q, W), vec(Q, 1.0, 0.2), mat(H * d, Q, 1.5)
            if m.get("kv_from") is None:
                w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(R, W), vec(R, 1.0, 0.2)
            w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * d, R, 1.5), mat(H * dv, R)
            w[p + "mix.sink"], w[p + "mix.g"] = vec(H, 0.5, 1.0), mat(H, W, 2.0)
            w[p + "mix.o"] = mat(W, H * dv)
        if lc.get("mlp"):
            norm(p + "norm2", 0.7)
            norm(p + "norm2b", 1.0)
            w[p + "mlp.up"], w[p + "mlp.down"] = mat(lc["mlp"]["ff"], W, 1.5), mat(W, lc["mlp"]["ff"])
        if sd:
            w[p + "side.gate"], w[p + "side.proj"], w[p + "side.norm"] = mat(sd, W, 1.5), mat(W, sd), vec(W, 1.0, 0.2)
    return w
