"""Plain, slow restatement of the Gekazen equations in float64, one function per mechanism.  It shares no code with the
package: it reads the family's configuration dictionary and a checkpoint dictionary with the family's tensor names
(``embed``, ``l<i>.mix.q`` ..., linear weights ``[out, in]``) and loops over tokens, heads and experts."""
import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def zero_centred_norm(x, w, eps):
    return unit_rms(x, eps) * (1.0 + w)


def slope(h, n_heads):
    return 2.0 ** (-8.0 * (h + 1) / n_heads)


def visible(i, j, size, keep_first):
    if j > i:
        return False
    if size is None:
        return True
    return (i - j < size) or (j < keep_first)


def attention_one_head(q, k, v, h, n_heads, scale, size, keep_first, q_positions=None):
    """q [Tq, D] at ``q_positions`` (default 0..Tq-1), k [Tk, D], v [Tk, Dv] at positions 0..Tk-1 -> [Tq, Dv]."""
    Tq, Tk = q.shape[0], k.shape[0]
    pos = list(range(Tq)) if q_positions is None else list(q_positions)
    out = torch.zeros(Tq, v.shape[1], dtype=F64)
    for a, i in enumerate(pos):
        js = [j for j in range(Tk) if visible(i, j, size, keep_first)]
        if not js:
            continue
        s = torch.stack([(q[a] * k[j]).sum() * scale - slope(h, n_heads) * (i - j) for j in js])
        p = torch.softmax(s, 0)
        out[a] = sum(p[n] * v[j] for n, j in enumerate(js))
    return out


def attention_vectorised(q, k, v, n_heads, kv_heads, scale, size, keep_first):
    """All heads of one sequence at once (same equations, matrix form; for the longer sequences).  q [T, H, D],
    k [T, G, D], v [T, G, Dv] -> [T, H, Dv]."""
    T = q.shape[0]
    i = torch.arange(T).reshape(T, 1)
    j = torch.arange(T).reshape(1, T)
    vis = j <= i
    if size is not None:
        vis = vis & ((i - j < size) | (j < keep_first))
    outs = []
    for h in range(n_heads):
        g = h // (n_heads // kv_heads)
        s = (q[:, h] @ k[:, g].T) * scale - slope(h, n_heads) * (i - j).to(F64)
        s = s.masked_fill(~vis, float("-inf"))
        outs.append(torch.softmax(s, -1) @ v[:, g])
    return torch.stack(outs, 1)


def expert(h, gate_w, up_w, down_w, limit):
    g = torch.clamp(h @ gate_w.T, max=limit)
    u = torch.clamp(h @ up_w.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down_w.T


def route(h, router_w, correction, top):
    """Scores and the chosen experts of one token."""
    s = torch.softmax(router_w @ h, 0)
    choice = s + correction
    chosen = sorted(range(len(s)), key=lambda e: (-float(choice[e]), e))[:top]
    return s, chosen


def moe(h, W, prefix, mlp):
    """h [T, width] -> [T, width]."""
    r = mlp["router"]
    E, I, top, scale = r["experts"], r.get("identity", 0), r["top"], r.get("scale", 1.0)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        s, chosen = route(h[t], W[prefix + "router"], W[prefix + "correction"], top)
        for e in chosen:
            w = s[e] * scale
            if e >= E:
                y[t] += w * h[t]
            else:
                y[t] += w * expert(h[t], W[f"{prefix}e{e}.gate"], W[f"{prefix}e{e}.up"], W[f"{prefix}e{e}.down"],
                                   mlp["expert"]["limit"])
        if mlp.get("shared"):
            gate = torch.sigmoid(W[prefix + "shared.sg"].reshape(-1) @ h[t])
            y[t] += gate * expert(h[t], W[prefix + "shared.gate"], W[prefix + "shared.up"], W[prefix + "shared.down"],
                                  mlp["shared"]["limit"])
    return y


def forward(cfg, weights, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence, float64."""
    W = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)]
    T = len(tokens)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        q = unit_rms((x @ W[p + "mix.q"].T + W[p + "mix.q.b"]).reshape(T, H, D), eps)
        if m.get("kv_from") is not None:
            k, v = kept[m["kv_from"]]
        else:
            k = unit_rms((x @ W[p + "mix.k"].T + W[p + "mix.k.b"]).reshape(T, G, D), eps)
            v = (x @ W[p + "mix.v"].T + W[p + "mix.v.b"]).reshape(T, G, Dv)
            kept[i] = (k, v)
        mask = m.get("mask") or {}
        o = attention_vectorised(q, k, v, H, G, m["scale"], mask.get("size"), mask.get("keep_first", 0))
        o = o.reshape(T, H * Dv) @ W[p + "mix.o"].T + W[p + "mix.o.b"]
        x = x + zero_centred_norm(o, W[p + "norm1"], eps)
        if layer.get("mlp"):
            x = x + zero_centred_norm(moe(x, W, p + "mlp.", layer["mlp"]), W[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return zero_centred_norm(x, W["final.norm"], eps) @ W["head"].T


def random_weights(cfg, seed=0, dtype=torch.float32, std=0.35):
    """A checkpoint dictionary with the family's tensor names for ``cfg``; values are rounded to bf16 so that a bf16
    and an fp32 model hold the same numbers."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=std):
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).to(dtype)

    Wd, V = cfg["width"], cfg["vocab"]
    sd = {"embed": rnd(V, Wd, s=1.0), "head": rnd(V, Wd, s=1.0 / math.sqrt(Wd)), "final.norm": rnd(Wd, s=0.1)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        lin = 1.0 / math.sqrt(Wd)
        sd[p + "mix.q"], sd[p + "mix.q.b"] = rnd(H * D, Wd, s=lin), rnd(H * D, s=0.1)
        if m.get("kv_from") is None:
            sd[p + "mix.k"], sd[p + "mix.k.b"] = rnd(G * D, Wd, s=lin), rnd(G * D, s=0.1)
            sd[p + "mix.v"], sd[p + "mix.v.b"] = rnd(G * Dv, Wd, s=lin), rnd(G * Dv, s=0.1)
        sd[p + "mix.o"], sd[p + "mix.o.b"] = rnd(Wd, H * Dv, s=1.0 / math.sqrt(H * Dv)), rnd(Wd, s=0.1)
        sd[p + "norm1"] = rnd(Wd, s=0.1)
        mlp = layer.get("mlp")
        if not mlp:
            continue
        sd[p + "norm2"] = rnd(Wd, s=0.1)
        r = mlp["router"]
        R = r["experts"] + r.get("identity", 0)
        sd[p + "mlp.router"], sd[p + "mlp.correction"] = rnd(R, Wd, s=0.5), rnd(R, s=0.05)
        F = mlp["expert"]["ff"]
        for e in range(r["experts"]):
            sd[f"{p}mlp.e{e}.gate"], sd[f"{p}mlp.e{e}.up"] = rnd(F, Wd, s=2 * lin), rnd(F, Wd, s=2 * lin)
            sd[f"{p}mlp.e{e}.down"] = rnd(Wd, F, s=1.0 / math.sqrt(F))
        if mlp.get("shared"):
            Fs = mlp["shared"]["ff"]
            sd[p + "mlp.shared.gate"], sd[p + "mlp.shared.up"] = rnd(Fs, Wd, s=2 * lin), rnd(Fs, Wd, s=2 * lin)
            sd[p + "mlp.shared.down"], sd[p + "mlp.shared.sg"] = rnd(Wd, Fs, s=1.0 / math.sqrt(Fs)), rnd(1, Wd, s=lin)
    return sd
