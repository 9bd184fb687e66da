"""Plain float64 restatement of the Vugipel design, one function per mechanism, for the tests. It shares no code with the engine.

A model is (cfg, weights): cfg is the config.json tree, weights maps tensor names to torch tensors. x [T, W] is the residual stream of T
tokens of one sequence at positions 0 .. T-1.

  layer:       x <- x + mixer(n1(x));  x <- x + ff(n2(x));   n(x) = x / sqrt(mean(x^2) + eps) * (1 + w)
  mingru:      z = sigmoid(Wz h + bz), u = Wx h + bx, c = u + 1/2 (u >= 0) | sigmoid(u) (u < 0)
               S_t = (1 - z_t) S_(t-1) + z_t c_t,  out = Wo (S_t * silu(Wg h))
  parallel:    left_scale * window_attention(h) + right_scale * retention(h)
  attention:   q, k = rope(headnorm(W h + b)), v = rot_p(Wv h + bv) over all value channels; s = softcap * tanh(scale * temp_h * q.k / softcap);
               key j visible to i when j <= i and (i - j < size or j < keep_first); softmax; out_i = rot_(-i)(sum_j p_ij v_j); Wo . + bo
  retention:   S_t = decay_h S_(t-1) + (k_t / sqrt(dim)) v_t^T,  o_t = S_t^T q_t;  Wo (unit_rms(o_t per head) * silu(Wg h))
  experts:     s = sigmoid(Wr h); the `top` largest; out = sum_e expert_e(s_e * h),  expert(y) = Wd (silu(Wg y) * (Wu y))
  readout:     head . n_final(x)
"""
import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is the distance from one"""
    return unit_rms(x, eps) * (1.0 + w.to(F64))


def silu(x):
    return x * torch.sigmoid(x)


def rotate_pairs(x, positions, base, dims, sign=1.0):
    """x [T, ..., n]: channels (2i, 2i+1), i < dims/2, turn by sign * p * base^(-2i/dims); channels from `dims` on pass unchanged."""
    x = x.to(F64)
    p = torch.as_tensor(positions, dtype=F64)
    i = torch.arange(dims // 2, dtype=F64)
    ang = sign * p[:, None] * base ** (-2.0 * i / dims)            # [T, dims/2]
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (dims // 2,)
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def min_gru_scan(z_logit, u, state):
    """z_logit, u [T, n]; state [n] -> (S [T, n], last state)"""
    z = torch.sigmoid(z_logit.to(F64))
    u = u.to(F64)
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = state.to(F64).clone()
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        out[t] = S
    return out, S


def min_gru_mixer(h, W, p, state):
    h = h.to(F64)
    zl = h @ W[p + "mix.z"].to(F64).T + W[p + "mix.z.b"].to(F64)
    u = h @ W[p + "mix.x"].to(F64).T + W[p + "mix.x.b"].to(F64)
    S, last = min_gru_scan(zl, u, state)
    g = h @ W[p + "mix.g"].to(F64).T
    return (S * silu(g)) @ W[p + "mix.o"].to(F64).T, last


def visible(i, j, size, keep_first):
    return j <= i and (i - j < size or j < keep_first)


def window_softmax_attention(q, k, v, pos_q, pos_k, heads, kv_heads, scale, temp, softcap, size, keep_first):
    """q [Tq, heads, dim], k [Tk, kv_heads, dim], v [Tk, kv_heads, vdim] -> [Tq, heads, vdim]"""
    Tq, Tk = q.shape[0], k.shape[0]
    per = heads // kv_heads
    pq, pk = torch.as_tensor(pos_q, dtype=torch.int64)[:, None], torch.as_tensor(pos_k, dtype=torch.int64)[None, :]
    mask = (pk <= pq) & ((pq - pk < size) | (pk < keep_first))          # visible(i, j, ...) for all pairs at once
    out = torch.zeros(Tq, heads, v.shape[-1], dtype=F64)
    for h in range(heads):
        g = h // per
        s = (q[:, h].to(F64) @ k[:, g].to(F64).T) * scale * float(temp[h])
        s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~mask, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g].to(F64)
    return out


def attention_cache_rows(h, W, p, mc, eps, positions):
    """What the left mixer keeps per token: normed rotated keys and rotated values."""
    h = h.to(F64)
    T = h.shape[0]
    k = (h @ W[p + "k"].to(F64).T + W[p + "k.b"].to(F64)).reshape(T, mc["kv_heads"], mc["dim"])
    k = unit_rms(k, eps) * W[p + "k.norm"].to(F64)
    k = rotate_pairs(k, positions, mc["rot"]["base"], mc["rot"]["dims"])
    v = (h @ W[p + "v"].to(F64).T + W[p + "v.b"].to(F64)).reshape(T, mc["kv_heads"], mc["vdim"])
    v = rotate_pairs(v, positions, mc["rot"]["base"], mc["vdim"])
    return k, v


def attention_mixer(h, W, p, mc, eps, positions, cache):
    """cache = (k, v, positions_k) of every earlier token of the sequence and of these"""
    h = h.to(F64)
    T = h.shape[0]
    q = (h @ W[p + "q"].to(F64).T + W[p + "q.b"].to(F64)).reshape(T, mc["heads"], mc["dim"])
    q = unit_rms(q, eps) * W[p + "q.norm"].to(F64)
    q = rotate_pairs(q, positions, mc["rot"]["base"], mc["rot"]["dims"])
    k, v, pk = cache
    o = window_softmax_attention(q, k, v, positions, pk, mc["heads"], mc["kv_heads"], mc["scale"], W[p + "temp"], mc["softcap"],
                                 mc["mask"]["size"], mc["mask"]["keep_first"])
    o = rotate_pairs(o, positions, mc["rot"]["base"], mc["vdim"], sign=-1.0)
    return o.reshape(T, -1) @ W[p + "o"].to(F64).T + W[p + "o.b"].to(F64)


def retention_scan(q, k, v, decay, state):
    """q, k [T, H, dim], v [T, H, vdim], decay [H], state [H, dim, vdim] -> (o [T, H, vdim], last state)"""
    T, H, dim = q.shape
    S = state.to(F64).clone()
    d = torch.as_tensor(decay, dtype=F64)[:, None, None]
    k = k.to(F64) / math.sqrt(dim)
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for t in range(T):
        S = d * S + k[t][:, :, None] * v[t].to(F64)[:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t].to(F64))
    return out, S


def retention_mixer(h, W, p, mc, eps, state):
    h = h.to(F64)
    T, H = h.shape[0], mc["heads"]
    q = (h @ W[p + "q"].to(F64).T).reshape(T, H, mc["dim"])
    k = (h @ W[p + "k"].to(F64).T).reshape(T, H, mc["dim"])
    v = (h @ W[p + "v"].to(F64).T).reshape(T, H, mc["vdim"])
    o, last = retention_scan(q, k, v, mc["decay"], state)
    o = unit_rms(o, eps).reshape(T, -1) * silu(h @ W[p + "g"].to(F64).T)
    return o @ W[p + "o"].to(F64).T, last


def routed_experts(h, W, p, ml):
    h = h.to(F64)
    n, top = ml["router"]["experts"], ml["router"]["top"]
    s = torch.sigmoid(h @ W[p + "router"].to(F64).T)
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        order = sorted(range(n), key=lambda e: (-float(s[t, e]), e))[:top]
        for e in order:
            y = s[t, e] * h[t]
            q = p + "e%d." % e
            out[t] += W[q + "down"].to(F64) @ (silu(W[q + "gate"].to(F64) @ y) * (W[q + "up"].to(F64) @ y))
    return out


class State:
    """What a sequence carries from token to token"""

    def __init__(self, cfg):
        self.pos = 0
        self.layers = []
        for lc in cfg["layers"]:
            mc = lc["mixer"]
            if lc["type"] == "mingru":
                self.layers.append({"s": torch.zeros(mc["width"], dtype=F64)})
            else:
                L, R = mc["left"], mc["right"]
                self.layers.append({"k": torch.zeros(0, L["kv_heads"], L["dim"], dtype=F64), "v": torch.zeros(0, L["kv_heads"], L["vdim"], dtype=F64),
                                    "s": torch.zeros(R["heads"], R["dim"], R["vdim"], dtype=F64)})


def forward(cfg, W, tokens, state=None, layer_outputs=None):
    """Next tokens of one sequence -> logits [T, vocab] (float64); state is advanced in place."""
    state = state or State(cfg)
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = list(range(state.pos, state.pos + T))
    x = W["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.int64)]
    for i, lc in enumerate(cfg["layers"]):
        p = "l%d." % i
        st = state.layers[i]
        mc = lc["mixer"]
        h = offset_norm(x, W[p + "norm1"], eps)
        if lc["type"] == "mingru":
            y, st["s"] = min_gru_mixer(h, W, p, st["s"])
        elif lc["type"] == "parallel":
            k, v = attention_cache_rows(h, W, p + "mix.left.", mc["left"], eps, positions)
            st["k"], st["v"] = torch.cat([st["k"], k]), torch.cat([st["v"], v])
            left = attention_mixer(h, W, p + "mix.left.", mc["left"], eps, positions, (st["k"], st["v"], list(range(state.pos + T))))
            right, st["s"] = retention_mixer(h, W, p + "mix.right.", mc["right"], eps, st["s"])
            y = mc["left_scale"] * left + mc["right_scale"] * right
        else:
            raise ValueError(lc["type"])
        x = x + y
        if lc.get("mlp"):
            x = x + routed_experts(offset_norm(x, W[p + "norm2"], eps), W, p + "mlp.", lc["mlp"])
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    state.pos += T
    return offset_norm(x, W["final.norm"], eps) @ W["head"].to(F64).T


# ---- small configurations and random weights for the tests ----------------------------------------------------------------------------
def moe_mlp(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def mingru_layer(width, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def parallel_layer(heads, kv_heads, dim, vdim, size, keep_first, r_heads, r_dim, r_vdim, decay, mlp=None, rot_dims=None, base=10000.0, scale=None,
                   softcap=15.0, left_scale=1.0, right_scale=1.0):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5),
            "softcap": float(softcap), "rot": {"base": float(base), "dims": dim if rot_dims is None else rot_dims},
            "mask": {"size": size, "keep_first": keep_first}}
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": [float(d) for d in decay]}
    return {"type": "parallel", "mixer": {"left": left, "left_scale": float(left_scale), "right": right, "right_scale": float(right_scale)}, "mlp": mlp}


def make_config(width, vocab, layers, eps=1e-6):
    return {"architecture": "Vugipel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


def random_weights(cfg, seed=0):
    """bf16 tensors (what a checkpoint holds), as a dict of torch tensors"""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def mat(rows, cols, gain=1.0):
        return (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vec(n, mean=0.0, spread=0.1):
        return (mean + spread * torch.randn(n, generator=g)).to(torch.bfloat16)

    t = {"embed": mat(V, W, math.sqrt(W)), "head": mat(V, W, 2.0), "final.norm": vec(W)}
    for i, lc in enumerate(cfg["layers"]):
        p = "l%d." % i
        mc = lc["mixer"]
        t[p + "norm1"] = vec(W, 0.0, 0.2)
        if lc["type"] == "mingru":
            n = mc["width"]
            t[p + "mix.z"], t[p + "mix.z.b"] = mat(n, W, 1.5), vec(n, 0.0, 0.7)
            t[p + "mix.x"], t[p + "mix.x.b"] = mat(n, W, 1.5), vec(n, 0.0, 0.7)
            t[p + "mix.g"], t[p + "mix.o"] = mat(n, W, 1.5), mat(W, n, 1.5)
        else:
            A, R = mc["left"], mc["right"]
            H, G, D, Dv = A["heads"], A["kv_heads"], A["dim"], A["vdim"]
            l, r = p + "mix.left.", p + "mix.right."
            t[l + "q"], t[l + "q.b"] = mat(H * D, W), vec(H * D, 0.0, 0.3)
            t[l + "k"], t[l + "k.b"] = mat(G * D, W), vec(G * D, 0.0, 0.3)
            t[l + "v"], t[l + "v.b"] = mat(G * Dv, W), vec(G * Dv, 0.0, 0.3)
            t[l + "q.norm"], t[l + "k.norm"] = vec(D, 1.0, 0.3), vec(D, 1.0, 0.3)
            t[l + "temp"] = (0.3 + torch.rand(H, generator=g) * 1.5).to(torch.bfloat16)
            t[l + "o"], t[l + "o.b"] = mat(W, H * Dv, 1.5), vec(W, 0.0, 0.2)
            Hr, Dr, Dvr = R["heads"], R["dim"], R["vdim"]
            t[r + "q"], t[r + "k"], t[r + "v"] = mat(Hr * Dr, W, 1.5), mat(Hr * Dr, W, 1.5), mat(Hr * Dvr, W)
            t[r + "g"], t[r + "o"] = mat(Hr * Dvr, W, 1.5), mat(W, Hr * Dvr, 1.5)
        ml = lc.get("mlp")
        if ml:
            t[p + "norm2"] = vec(W, 0.0, 0.2)
            f, E = ml["expert"]["ff"], ml["router"]["experts"]
            t[p + "mlp.router"] = mat(E, W, 3.0)
            for x in range(E):
                q = "%smlp.e%d." % (p, x)
                t[q + "gate"], t[q + "up"], t[q + "down"] = mat(f, W, 1.5), mat(f, W, 1.5), mat(W, f, 1.5)
    return t
