"""A plain, slow float64 implementation of the Rasodra family, one function per mechanism, working on whole sequences
(no cache, no state carried between calls, no batches).  It shares no code with the package: the tests compare the
framework's step function, cache, state and kernels against it.

Checkpoint names: ``embed``, ``l<i>.norm1 / norm1b / norm2 / norm2b``, ``l<i>.mix.<name>`` (``<name>.b`` for a bias),
``l<i>.mlp.up / down``, ``final.norm``, ``head``; linear weights are ``[out, in]``.
"""
import math

import torch

F64 = torch.float64


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate(x, positions, dims, base):
    """x [T, H, D]: pair (2i, 2i+1), i < dims/2, of the token at position p turns by p * base^(-2i/dims)."""
    out = x.clone()
    for i in range(dims // 2):
        ang = positions.to(F64) * base ** (-2.0 * i / dims)
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def softmax_rows(scores, visible, sink=None):
    """scores [H, T, T]; visible [T, T] bool; sink [H] or None: one more term exp(sink_h) in every denominator."""
    s = scores.masked_fill(~visible, -math.inf)
    mx = s.max(-1, keepdim=True).values
    if sink is not None:
        mx = torch.maximum(mx, sink.reshape(-1, 1, 1))
    e = torch.exp(s - mx)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.reshape(-1, 1, 1) - mx)
    return e / den


def chunked_attention(h, W, p, m, eps):
    T = h.shape[0]
    H, G, D = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, D)
    v = k.clone()                                                  # the raw key projections double as values
    q = unit_rms(q, eps) * W[p + "q.norm"]
    k = unit_rms(k, eps) * W[p + "k.norm"]
    pos = torch.arange(T)
    if m.get("rot"):
        q = rotate(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate(k, pos, m["rot"]["dims"], m["rot"]["base"])
    rep = H // G
    out = torch.zeros(T, H, D, dtype=F64)
    size = (m.get("mask") or {}).get("size")
    vis = pos[None, :] <= pos[:, None]
    if size:
        vis = vis & ((pos[:, None] // size) == (pos[None, :] // size))
    for hd in range(H):
        g = hd // rep
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        pr = softmax_rows(s[None], vis)[0]
        out[:, hd] = pr @ v[:, g]
    return out.reshape(T, H * D) @ W[p + "o"].T


def latent_attention(h, W, p, m, eps):
    T = h.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ W[p + "q"].T).reshape(T, H, D + R)
    dkv = h @ W[p + "dkv"].T
    c = unit_rms(dkv[:, :C], eps) * W[p + "dkv.norm"]
    pos = torch.arange(T)
    k_rot = rotate(dkv[:, C:].reshape(T, 1, R), pos, m["rot"]["dims"], m["rot"]["base"])[:, 0]
    q_rot = rotate(q[..., D:], pos, m["rot"]["dims"], m["rot"]["base"])
    k_nope = (c @ W[p + "uk"].T).reshape(T, H, D)
    v = (c @ W[p + "uv"].T).reshape(T, H, Dv)
    vis = pos[None, :] <= pos[:, None]
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        s = (q[:, hd, :D] @ k_nope[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        pr = softmax_rows(s[None], vis, W[p + "sink"][hd:hd + 1])[0]
        out[:, hd] = pr @ v[:, hd]
    gate = torch.sigmoid(h @ W[p + "g"].T)
    return (out.reshape(T, H * Dv) * gate) @ W[p + "o"].T


def mlstm_gates(h, W, p, m):
    cap = m["gate_cap"]
    i = cap * torch.tanh((h @ W[p + "i"].T + W[p + "i.b"]) / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ W[p + "f"].T + W[p + "f.b"]) / cap))
    return i, f


def mlstm_cell(q, k, v, i, f):
    """q, k [T, H, D] (q already scaled), v [T, H, Dv], gates [T, H] -> o [T, H, Dv]; zero state, m_0 = 0."""
    T, H, D = q.shape
    Dv = v.shape[-1]
    S = torch.zeros(H, D, Dv, dtype=F64)
    n = torch.zeros(H, D, dtype=F64)
    mx = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(f[t] + mx, i[t])
        a, b = torch.exp(f[t] + mx - m_new), torch.exp(i[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        mx = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    return out


def mlstm(h, W, p, m, eps):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, Dv)
    i, f = mlstm_gates(h, W, p, m)
    o = unit_rms(mlstm_cell(q, k, v, i, f), eps).reshape(T, H * Dv)
    o = o * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def feed_forward(h, W, p):
    return torch.relu(h @ W[p + "up"].T) ** 2 @ W[p + "down"].T


MIXERS = {"attention": chunked_attention, "latent_attention": latent_attention, "mlstm": mlstm}


def forward(cfg, sd, tokens, streams=None):
    """Logits [T, vocab] of one sequence; ``streams`` (a list) receives the residual stream after every layer."""
    W = {k: v.to(F64) for k, v in sd.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)]
    for i, L in enumerate(cfg["layers"]):
        j = L.get("weights_of")
        p = f"l{i if j is None else j}."
        x = x + layer_norm(MIXERS[L["type"]](layer_norm(x, W[p + "norm1"], eps), W, p + "mix.", L["mixer"], eps),
                           W[p + "norm1b"], eps)
        if L.get("mlp"):
            x = x + layer_norm(feed_forward(layer_norm(x, W[p + "norm2"], eps), W, p + "mlp."), W[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return layer_norm(x, W["final.norm"], eps) @ W["head"].T


def random_weights(cfg, seed=0, spread=1.0):
    """Checkpoint tensors for ``cfg`` (values exactly representable in bf16, so that every dtype loads the same model)."""
    g = torch.Generator().manual_seed(seed)
    Wd = cfg["width"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s * spread / math.sqrt(i)).to(torch.bfloat16).float()

    def vec(n, mean=0.0, s=1.0):
        return (mean + torch.randn(n, generator=g) * s).to(torch.bfloat16).float()

    sd = {"embed": vec(cfg["vocab"] * Wd).reshape(cfg["vocab"], Wd), "final.norm": vec(Wd, 1.0, 0.2),
          "head": mat(cfg["vocab"], Wd)}
    for i, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", L["mixer"]
        for n in ["norm1", "norm1b"] + (["norm2", "norm2b"] if L.get("mlp") else []):
            sd[p + n] = vec(Wd, 1.0, 0.2)
        H = m["heads"]
        if L["type"] == "attention":
            G, D = m.get("kv_heads", H), m["dim"]
            sd[p + "mix.q"], sd[p + "mix.k"] = mat(H * D, Wd, 2.0), mat(G * D, Wd, 2.0)
            sd[p + "mix.q.b"], sd[p + "mix.k.b"] = vec(H * D, 0.0, 0.3), vec(G * D, 0.0, 0.3)
            sd[p + "mix.q.norm"], sd[p + "mix.k.norm"] = vec(D, 1.0, 0.3), vec(D, 1.0, 0.3)
            sd[p + "mix.o"] = mat(Wd, H * D)
        elif L["type"] == "latent_attention":
            D, R, Dv, C = m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            sd[p + "mix.q"], sd[p + "mix.dkv"] = mat(H * (D + R), Wd, 2.0), mat(C + R, Wd, 2.0)
            sd[p + "mix.dkv.norm"] = vec(C, 1.0, 0.3)
            sd[p + "mix.uk"], sd[p + "mix.uv"] = mat(H * D, C, 2.0), mat(H * Dv, C)
            sd[p + "mix.sink"] = vec(H, 0.5, 1.0)
            sd[p + "mix.g"], sd[p + "mix.o"] = mat(H * Dv, Wd), mat(Wd, H * Dv)
        else:
            D, Dv = m["dim"], m["vdim"]
            sd[p + "mix.q"], sd[p + "mix.k"], sd[p + "mix.v"] = mat(H * D, Wd, 2.0), mat(H * D, Wd, 2.0), mat(H * Dv, Wd)
            sd[p + "mix.g"], sd[p + "mix.o"] = mat(H * Dv, Wd), mat(Wd, H * Dv)
            sd[p + "mix.norm"] = vec(H * Dv, 1.0, 0.2)
            sd[p + "mix.i"], sd[p + "mix.f"] = mat(H, Wd, 3.0), mat(H, Wd, 3.0)
            sd[p + "mix.i.b"], sd[p + "mix.f.b"] = vec(H, -1.0, 1.0), vec(H, 3.0, 1.5)
        if L.get("mlp"):
            sd[p + "mlp.up"], sd[p + "mlp.down"] = mat(L["mlp"]["ff"], Wd, 1.5), mat(Wd, L["mlp"]["ff"])
    return sd
