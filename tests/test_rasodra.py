"""Rasodra family against the float64 oracle of ``tests/rasodra_oracle.py``: every mechanism alone, then the model through
the framework's step function, cache / state manager and schedulers.  Every test runs on the CPU (the ops' PyTorch
path) and, marked ``gpu``, on CUDA (the kernels) in fp32 and bf16."""
import json
import os
import subprocess
import sys

import pytest
import torch

import rasodra_oracle as O
from neuronx_distributed_llama3_2_b200.inference import InferenceConfig, RasodraInferenceModel
from neuronx_distributed_llama3_2_b200.inference.kv_cache import KVCache
from neuronx_distributed_llama3_2_b200.inference.trace_replay import TraceReplayer
from neuronx_distributed_llama3_2_b200.models.rasodra import (RasodraConfig, convert_rasodra_state_dict,
                                                              export_rasodra_state_dict, tiny_rasodra)
from neuronx_distributed_llama3_2_b200.ops import activation as act_ops
from neuronx_distributed_llama3_2_b200.ops import latent_attention as la
from neuronx_distributed_llama3_2_b200.ops import mlstm as ml
from neuronx_distributed_llama3_2_b200.ops import norm as norm_ops
from neuronx_distributed_llama3_2_b200.ops import rope as rope_ops
from neuronx_distributed_llama3_2_b200.ops import window_attention as wa

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F64 = torch.float64
CASES = [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu),
         pytest.param("cuda", torch.bfloat16, marks=pytest.mark.gpu)]
case = pytest.mark.parametrize("dev,dt", CASES)


def tol(dt):
    return 2e-4 if dt == torch.float32 else 6e-2


def close(a, b, dt, scale=1.0):
    err = (a.detach().to("cpu", F64) - b.to(F64)).abs().max().item()
    assert err <= tol(dt) * scale, f"max error {err:.3e} above {tol(dt) * scale:.1e}"


ATT = dict(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.3, mask={"size": 8}, rot={"dims": 8, "base": 10000.0})
LAT = dict(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=24, scale=0.25, rot={"dims": 4, "base": 5000.0})
REC = dict(heads=2, dim=12, vdim=20, gate_cap=9.0)
FF = {"kind": "dense", "ff": 56}


def layer(kind, mlp=FF, weights_of=None, **kw):
    m = dict({"attention": ATT, "latent_attention": LAT, "mlstm": REC}[kind])
    m.update(kw)
    d = {"type": kind, "mixer": m, "mlp": mlp}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def config(layers=None, vocab=96, width=40):
    layers = layers or [layer("attention"), layer("mlstm", mlp=None), layer("latent_attention"),
                        layer("mlstm", mlp=None, weights_of=1), layer("attention", weights_of=0),
                        layer("latent_attention", weights_of=2)]
    return {"architecture": "Rasodra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": layers}


# what the usual configurations make equal or 1: a single head, as many key/value heads as heads, rotation over all and
# over two dimensions, a chunk of one position and no chunks, a recurrent first layer, a feed-forward after the
# recurrent layer and none after attention, no layer that borrows weights, odd sizes
ODD = config(layers=[
    layer("mlstm", heads=1, dim=5, vdim=7, gate_cap=3.0),
    layer("attention", mlp=None, heads=3, kv_heads=3, dim=6, vdim=6, mask={"size": 1}, rot={"dims": 6, "base": 100.0}),
    layer("latent_attention", mlp=None, heads=1, dim=6, rot_dim=2, vdim=5, kv_rank=9, rot={"dims": 2, "base": 77.0}),
    layer("attention", heads=6, kv_heads=1, dim=10, vdim=10, mask=None, rot={"dims": 2, "base": 9.0}),
    layer("mlstm", mlp=None, heads=3, dim=33, vdim=35, gate_cap=20.0),
], vocab=50, width=30)


def build(cfg, dev, dt, lines=4, seq_len=96, seed=0, paged=False, pages=None, page_size=8, sd=None):
    sd = sd if sd is not None else O.random_weights(cfg, seed)
    rc = RasodraConfig.from_dict(cfg, torch_dtype=dt)
    ic = InferenceConfig(batch_size=lines, max_batch_size=lines, max_context_length=seq_len, seq_len=seq_len,
                         is_continuous_batching=True, use_cuda_graphs=False, paged_kv=paged, page_size=page_size,
                         num_kv_pages=pages)
    model = RasodraInferenceModel(rc, ic, device=torch.device(dev))
    missing, unexpected = model.load_state_dict(convert_rasodra_state_dict(sd, rc), strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    model.init_kv_cache(device=torch.device(dev))
    return model, sd


def tokens_of(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def replay(model, steps):
    rp = TraceReplayer(model)
    got = {}
    for entries, end in steps:
        out = rp.step(entries, end)
        r = 0
        for e in entries:
            for _ in e["want"]:
                got.setdefault(e["id"], []).append(out[r].cpu())
                r += 1
    return got


def check_rows(rows, ref, places, dt):
    """Every position against the oracle: centred difference over the vocabulary, relative to the spread of the logits.
    fp32 is strict.  bf16 rounding through six tiny layers reaches a few percent at single positions (the PyTorch bf16
    path of the same ops shows the same), so bf16 bounds every position at 0.2 and the mean over positions at 0.04; a
    wrong key, edge or state moves positions by far more."""
    assert len(rows) == len(places)
    rels = []
    for row, p in zip(rows, places):
        d = row.to(F64) - ref[p]
        d = d - d.mean()
        rel = float(d.pow(2).mean().sqrt() / ref[p].std())
        assert rel <= (2e-4 if dt == torch.float32 else 0.2), f"position {p}: relative error {rel:.2e}"
        rels.append(rel)
    assert dt == torch.float32 or sum(rels) / len(rels) <= 0.04, f"mean relative error {sum(rels) / len(rels):.2e}"


# ---- mechanisms alone ---------------------------------------------------------------------------------------------------
@case
def test_qk_norm_rotation_and_cache_write(dev, dt):
    """Weighted per-head norm, pairwise rotation of the first dims only, cached value = the raw key projection."""
    torch.manual_seed(1)
    B, T, H, G, D, S, rot = 2, 9, 4, 2, 10, 40, 6
    qk = torch.randn(B, T, (H + G) * D)
    qw, kw = torch.randn(D), torch.randn(D)
    ck, cv = torch.zeros(3, G, S, D, dtype=dt, device=dev), torch.zeros(3, G, S, D, dtype=dt, device=dev)
    start, n_new, lines = torch.tensor([0, 23]), torch.tensor([9, 5]), torch.tensor([2, 0])
    tables = rope_ops.build_interleaved_rope_cache(S, rot, 50.0, device=dev)
    q = wa.qk_norm_cache_write(qk.to(dev, dt), ck, cv, start.to(dev), H, G, D, D, 1e-6, n_new=n_new.to(dev),
                               seq_ids=lines.to(dev), q_weight=qw.to(dev), k_weight=kw.to(dev), rope=tables,
                               value_from_key=True)
    x = qk.to(dt).to(F64)
    for b in range(B):
        n, s, ln = int(n_new[b]), int(start[b]), int(lines[b])
        pos = torch.arange(s, s + T)
        qr = O.rotate(O.unit_rms(x[b, :, :H * D].reshape(T, H, D), 1e-6) * qw.to(F64), pos, rot, 50.0)
        close(q[b, :n], qr[:n], dt, scale=3.0)
        kraw = x[b, :, H * D:].reshape(T, G, D)
        kr = O.rotate(O.unit_rms(kraw, 1e-6) * kw.to(F64), pos, rot, 50.0)
        close(ck[ln, :, s:s + n], kr[:n].transpose(0, 1), dt, scale=3.0)
        close(cv[ln, :, s:s + n], kraw[:n].transpose(0, 1), dt)
        assert float(ck[ln, :, s + n:].abs().sum()) == 0.0 and float(ck[ln, :, :s].abs().sum()) == 0.0
    assert float(ck[1].abs().sum()) == 0.0
    # dimensions past the rotated ones pass unchanged
    close(q[0, :, :, rot:], (O.unit_rms(x[0, :, :H * D].reshape(T, H, D), 1e-6) * qw.to(F64))[..., rot:], dt, scale=3.0)


def _attention_oracle(q, k, v, q_pos, scale, chunk=None, sink=None):
    """q [Tq, H, D] at positions q_pos over keys [G, Tk, D] / values [G, Tk, Dv]."""
    H, G = q.shape[1], k.shape[0]
    out = torch.zeros(q.shape[0], H, v.shape[-1], dtype=F64)
    j = torch.arange(k.shape[1])
    for t in range(q.shape[0]):
        p = int(q_pos[t])
        vis = j <= p
        if chunk:
            vis = vis & ((j // chunk) == (p // chunk))
        for hd in range(H):
            g = hd // (H // G)
            s = (k[g].to(F64) @ q[t, hd].to(F64)) * scale
            s = s.masked_fill(~vis, float("-inf"))
            mx = s.max() if sink is None else torch.maximum(s.max(), sink[hd].to(F64))
            e = torch.exp(s - mx)
            den = e.sum() + (torch.exp(sink[hd].to(F64) - mx) if sink is not None else 0.0)
            out[t, hd] = (e / den) @ v[g].to(F64)
    return out


@case
@pytest.mark.parametrize("paged", [False, True], ids=["contiguous", "paged"])
@pytest.mark.parametrize("D", [16, 32, 64], ids=["d16", "d32", "d64"])
@pytest.mark.parametrize("chunk,sink", [(8, False), (5, True), (None, True), (64, False), (48, True), (100, False)])
def test_attention_over_the_cache_chunks_and_sinks(dev, dt, paged, chunk, sink, D):
    """Prompt portion at an offset and single-token decoding; one key just inside and one just outside the query's chunk
    carry a score that dominates, so a chunk edge that is one token off changes the result."""
    torch.manual_seed(3)
    H, G, Dv, S, page = 4, 2, D, 160, 8                 # head sizes 32 and 64 take the tensor-core kernels in bf16
    start, T = 101, 37
    n_ctx = start + T
    k = torch.randn(G, n_ctx, D).to(dt)
    v = torch.randn(G, n_ctx, Dv).to(dt)
    q = torch.randn(T, H, D).to(dt)
    if chunk:
        edge = ((start + T - 1) // chunk) * chunk                 # first position of the last query's chunk
        if edge >= 1:
            k[:, edge] = q[T - 1, 0] * 2.0                           # just inside: dominates that query's softmax
            k[:, edge - 1] = q[T - 1, 0] * 3.0                       # just outside: must not be seen
    sinks = torch.tensor([0.5, -1.0, 3.0, 6.0]) if sink else None
    if paged:
        g = torch.Generator().manual_seed(5)
        table = torch.randperm(40, generator=g).to(torch.int32).reshape(2, 20)
        ck, cv = torch.zeros(40, G, page, D, dtype=dt), torch.zeros(40, G, page, Dv, dtype=dt)
        for pos in range(n_ctx):
            ck[table[1, pos // page], :, pos % page], cv[table[1, pos // page], :, pos % page] = k[:, pos], v[:, pos]
        kw = dict(block_table=table.to(dev), page_size=page)
    else:
        ck, cv = torch.zeros(3, G, S, D, dtype=dt), torch.zeros(3, G, S, Dv, dtype=dt)
        ck[1, :, :n_ctx], cv[1, :, :n_ctx] = k, v
        kw = {}
    ck, cv = ck.to(dev), cv.to(dev)
    sk = sinks.to(dev) if sink else None
    scale = 0.3 * (16 / D) ** 0.5
    ref = _attention_oracle(q, k, v, torch.arange(start, n_ctx), scale, chunk, sinks)
    line = torch.tensor([1], dtype=torch.int32, device=dev)
    out = wa.window_attention_prefill(q[None].to(dev), ck, cv, torch.tensor([start], device=dev), scale, seq_ids=line,
                                      chunk=chunk, sinks=sk, **kw)
    close(out[0], ref, dt)
    one = wa.window_attention_decode(q[T - 1:T].to(dev), ck, cv, torch.tensor([n_ctx - 1], device=dev), scale,
                                     seq_ids=line, chunk=chunk, sinks=sk, **kw)
    close(one[0], ref[T - 1], dt)
    if chunk and edge >= 1:
        seen_outside = _attention_oracle(q[T - 1:], k, v, torch.tensor([n_ctx - 1]), scale, None, sinks)
        assert float((seen_outside[0] - ref[T - 1]).abs().max()) > 0.05


@case
@pytest.mark.parametrize("D,Dv", [(288, 256), (576, 512), (40, 24)], ids=["288", "576", "40"])
def test_wide_latent_rows_one_tensor_for_keys_and_values(dev, dt, D, Dv):
    """One key/value head whose value is the first Dv columns of its D-column key rows (the latent cache), twenty query
    heads, a sink per head: token generation over a cache line and a prompt portion at an offset."""
    torch.manual_seed(12)
    H, S, n_ctx = 20, 160, 150
    rows = (torch.randn(n_ctx, D) * 0.5).to(dt)
    cache = torch.zeros(2, 1, S, D, dtype=dt)
    cache[1, 0, :n_ctx] = rows
    cache = cache.to(dev)
    q = (torch.randn(9, H, D) * 0.5).to(dt)
    sinks = torch.randn(H)
    line = torch.tensor([1], dtype=torch.int32, device=dev)
    ref = _attention_oracle(q, rows[None], rows[None, :, :Dv], torch.arange(n_ctx - 9, n_ctx), 0.1, None, sinks)
    one = wa.window_attention_decode(q[8:9].to(dev), cache, cache[..., :Dv], torch.tensor([n_ctx - 1], device=dev), 0.1,
                                     seq_ids=line, sinks=sinks.to(dev))
    close(one[0], ref[8], dt)
    part = wa.window_attention_prefill(q[None].to(dev), cache, cache[..., :Dv], torch.tensor([n_ctx - 9], device=dev), 0.1,
                                       seq_ids=line, sinks=sinks.to(dev))
    close(part[0], ref, dt)
    # three rows of different lengths on a paged cache, with the context split over CTAs and in one piece
    page, lens, lines3 = 16, [150, 70, 5], [1, 0, 2]
    g = torch.Generator().manual_seed(3)
    table = torch.randperm(30, generator=g).to(torch.int32).reshape(3, 10)
    paged = torch.zeros(30, 1, page, D, dtype=dt)
    seqs = [(torch.randn(n, D, generator=g) * 0.5).to(dt) for n in lens]
    for ln, rows_ in zip(lines3, seqs):
        for pos in range(rows_.shape[0]):
            paged[table[ln, pos // page], 0, pos % page] = rows_[pos]
    paged = paged.to(dev)
    q3 = (torch.randn(3, H, D, generator=g) * 0.5).to(dt)
    want = torch.stack([_attention_oracle(q3[i:i + 1], seqs[i][None], seqs[i][None, :, :Dv], torch.tensor([lens[i] - 1]), 0.1,
                                          None, sinks)[0] for i in range(3)])
    from neuronx_distributed_llama3_2_b200.ops import latent_attention as la_mod

    for target in (la_mod.TARGET_CTAS, 1):
        old, la_mod.TARGET_CTAS = la_mod.TARGET_CTAS, target
        try:
            got = wa.window_attention_decode(q3.to(dev), paged, paged[..., :Dv], torch.tensor([n - 1 for n in lens], device=dev),
                                             0.1, seq_ids=torch.tensor(lines3, dtype=torch.int32, device=dev),
                                             sinks=sinks.to(dev), block_table=table.to(dev), page_size=page)
        finally:
            la_mod.TARGET_CTAS = old
        close(got, want, dt)


@case
def test_expanded_latent_heads_of_192_and_128(dev, dt):
    """Prompt attention over per-head expanded keys of 192 and values of 128 columns read through strided views (the
    layout the latent mixer builds: [rows, positions, heads, columns]), with sinks and padding rows."""
    torch.manual_seed(13)
    B, T, H, D, Dv = 2, 70, 3, 192, 128
    q = (torch.randn(B, T, H, D) * 0.3).to(dt)
    keys = (torch.randn(B, T, H, D) * 0.3).to(dt)
    vals = torch.randn(B, T, H, Dv).to(dt)
    sinks = torch.tensor([0.0, 2.0, -1.0])
    n_new = torch.tensor([70, 33])
    out = wa.window_attention_prefill(q.to(dev), keys.to(dev).permute(0, 2, 1, 3), vals.to(dev).permute(0, 2, 1, 3),
                                      torch.zeros(B, dtype=torch.int32, device=dev), 0.2, n_new=n_new.to(dev),
                                      sinks=sinks.to(dev))
    for b in range(B):
        n = int(n_new[b])
        ref = _attention_oracle(q[b, :n], keys[b, :n].transpose(0, 1), vals[b, :n].transpose(0, 1), torch.arange(n), 0.2,
                                None, sinks)
        close(out[b, :n], ref, dt)
        assert float(out[b, n:].abs().sum()) == 0.0


@case
def test_latent_rows_and_absorbed_queries_equal_expanded_keys_and_values(dev, dt):
    """The cache keeps [norm(c) | rotated key part]; attention with absorbed queries over those rows followed by the
    value up-projection equals attention over per-head expanded keys and values."""
    torch.manual_seed(4)
    m = dict(LAT, heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=24)
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    Wd, T = 20, 13
    cfg = config(layers=[layer("latent_attention", mlp=None, **m)], width=Wd)
    sd = O.random_weights(cfg, 5)
    W = {k: v.to(F64) for k, v in sd.items()}
    h = torch.randn(T, Wd).to(dt)
    ref = O.latent_attention(h.to(F64), W, "l0.mix.", cfg["layers"][0]["mixer"], 1e-6)       # [T, width] after W_o
    proj = (h.to(F64) @ torch.cat([W["l0.mix.q"], W["l0.mix.dkv"], W["l0.mix.g"]]).T).to(dt)[None].to(dev).contiguous()
    cache = torch.zeros(2, 1, 32, C + R, dtype=dt, device=dev)
    q_abs = torch.zeros(T, H, C + R, dtype=dt, device=dev)
    tables = rope_ops.build_interleaved_rope_cache(32, R, m["rot"]["base"], device=dev)
    line = torch.tensor([1], dtype=torch.int32, device=dev)
    q_nope = la.latent_prep(proj, 0, H * (D + R), q_abs, cache, sd["l0.mix.dkv.norm"].to(dev), tables,
                            torch.tensor([0], device=dev), H, D, R, C, 1e-6, seq_ids=line)
    c_ref = O.unit_rms(proj[0].to("cpu", F64)[:, H * (D + R): H * (D + R) + C], 1e-6) * W["l0.mix.dkv.norm"]
    close(cache[1, 0, :T, :C], c_ref, dt, scale=3.0)
    assert float(cache[0].abs().sum()) == 0.0 and float(cache[1, 0, T:].abs().sum()) == 0.0
    uk = sd["l0.mix.uk"].reshape(H, D, C).to(dev, dt)
    q_abs[..., :C] = torch.bmm(q_nope.transpose(0, 1), uk).transpose(0, 1)
    o_lat = wa.window_attention_prefill(q_abs[None], cache, cache[..., :C], torch.tensor([0], device=dev), m["scale"],
                                        seq_ids=line, sinks=sd["l0.mix.sink"].to(dev))
    uv = sd["l0.mix.uv"].reshape(H, Dv, C).to(dev, dt)
    o = torch.bmm(o_lat[0].transpose(0, 1), uv.transpose(1, 2)).transpose(0, 1).contiguous()
    y = ml.head_norm_gate(o, proj[0], H * (D + R) + C + R, H, Dv, None, 1e-6, False, dt)
    close(y.to("cpu", F64) @ W["l0.mix.o"].T, ref, dt, scale=3.0)


@case
def test_recurrent_gates_scan_and_state(dev, dt):
    """Gates in fp32; the scan over a whole prompt equals the scan in portions of 1 / 3 / 17 tokens continued from the
    line's state; padding tokens leave the state alone; a row at position 0 ignores what its line held before."""
    torch.manual_seed(6)
    m = dict(REC, heads=2, dim=12, vdim=37, gate_cap=6.0)
    H, D, Dv, Wd, T = m["heads"], m["dim"], m["vdim"], 24, 45
    cfg = config(layers=[layer("mlstm", mlp=None, **m)], width=Wd)
    sd = O.random_weights(cfg, 7)
    W = {k: v.to(F64) for k, v in sd.items()}
    h = (torch.randn(T, Wd) * 2).to(dt)
    gi_ref, gf_ref = O.mlstm_gates(h.to(F64), W, "l0.mix.", m)
    gw = torch.cat([sd["l0.mix.i"], sd["l0.mix.f"]]).to(dev, dt)
    gb = torch.cat([sd["l0.mix.i.b"], sd["l0.mix.f.b"]]).to(dev)
    gi, gf = ml.mlstm_gates(h.to(dev), gw, gb, H, m["gate_cap"])
    assert gi.dtype == torch.float32 and gf.dtype == torch.float32
    close(gi, gi_ref, torch.float32, scale=0.5)
    close(gf, gf_ref, torch.float32, scale=0.5)
    proj = (h.to(F64) @ torch.cat([W["l0.mix.q"], W["l0.mix.k"], W["l0.mix.v"]]).T).to(dt)
    pf = proj.to(F64)
    ref = O.mlstm_cell(pf[:, :H * D].reshape(T, H, D) * D ** -0.5, pf[:, H * D:2 * H * D].reshape(T, H, D),
                       pf[:, 2 * H * D:].reshape(T, H, Dv), gi.to("cpu", F64), gf.to("cpu", F64))

    def state(fill=0.0):
        return (torch.full((3, H, D, Dv), fill, device=dev), torch.full((3, H, D), fill, device=dev),
                torch.full((3, H), fill, device=dev))

    offs = (0, H * D, 2 * H * D)
    line = torch.tensor([2], dtype=torch.int32, device=dev)
    st = state(fill=9.0)                                       # stale state of an earlier request on the same line
    whole = ml.mlstm_scan(proj[None].to(dev).contiguous(), offs, gi, gf, st, torch.tensor([0], device=dev), H, D, Dv,
                          D ** -0.5, seq_ids=line)
    close(whole[0], ref, torch.float32, scale=5.0)
    assert float((st[0][0] - 9.0).abs().max()) == 0.0         # other lines untouched
    st2 = state(fill=-3.0)
    got, lo = [], 0
    for n in (1, 3, 17, 1, 23):
        Tpad = n + 2                                           # two padding tokens behind every portion
        part = torch.zeros(1, Tpad, proj.shape[1], dtype=dt)
        part[0, :n] = proj[lo:lo + n]
        g_i, g_f = torch.zeros(Tpad, H), torch.full((Tpad, H), -50.0)
        g_i[:n], g_f[:n] = gi[lo:lo + n].cpu(), gf[lo:lo + n].cpu()
        o = ml.mlstm_scan(part.to(dev), offs, g_i.to(dev), g_f.to(dev), st2, torch.tensor([lo], device=dev), H, D, Dv,
                          D ** -0.5, n_new=torch.tensor([n], device=dev), seq_ids=line)
        got.append(o[0, :n])
        assert float(o[0, n:].abs().sum()) == 0.0
        lo += n
    close(torch.cat(got), ref, torch.float32, scale=5.0)
    for a, b in zip(st, st2):
        close(a[2], b[2].to("cpu", F64), torch.float32, scale=5.0)
    # token generation: 40 tokens at once, then one token per call (no padding mask) on the same line
    st5 = state(fill=2.0)
    ml.mlstm_scan(proj[None, :40].to(dev).contiguous(), offs, gi[:40], gf[:40], st5, torch.tensor([0], device=dev), H, D,
                  Dv, D ** -0.5, seq_ids=line)
    steps = [ml.mlstm_scan(proj[None, t:t + 1].to(dev).contiguous(), offs, gi[t:t + 1], gf[t:t + 1], st5,
                           torch.tensor([t], device=dev), H, D, Dv, D ** -0.5, seq_ids=line)[0, 0] for t in range(40, T)]
    close(torch.stack(steps), ref[40:], torch.float32, scale=5.0)
    for a, b in zip(st, st5):
        close(a[2], b[2].to("cpu", F64), torch.float32, scale=5.0)
    assert float((st5[0][1] - 2.0).abs().max()) == 0.0
    # the chunk-wise form: the whole prompt with chunks of 8 (five full chunks and a partial one), then two portions that
    # continue from the line's state, the second with padding behind it; same outputs, same final state
    st3 = state(fill=5.0)
    cw = ml.mlstm_chunkwise(proj[None].to(dev).contiguous(), offs, gi, gf, st3, torch.tensor([0], device=dev), H, D, Dv,
                            D ** -0.5, seq_ids=line, chunk=8)
    close(cw[0], ref, torch.float32, scale=5.0)
    for a, b in zip(st, st3):
        close(a[2], b[2].to("cpu", F64), torch.float32, scale=5.0)
    assert float((st3[0][0] - 5.0).abs().max()) == 0.0
    st4 = state(fill=1.0)
    first = ml.mlstm_chunkwise(proj[None, :19].to(dev).contiguous(), offs, gi[:19], gf[:19], st4,
                               torch.tensor([0], device=dev), H, D, Dv, D ** -0.5, seq_ids=line, chunk=16)
    part = torch.zeros(1, 30, proj.shape[1], dtype=dt)
    part[0, :26] = proj[19:]
    g_i, g_f = torch.zeros(30, H), torch.zeros(30, H)
    g_i[:26], g_f[:26] = gi[19:].cpu(), gf[19:].cpu()
    second = ml.mlstm_chunkwise(part.to(dev), offs, g_i.to(dev), g_f.to(dev), st4, torch.tensor([19], device=dev), H, D,
                                Dv, D ** -0.5, n_new=torch.tensor([26], device=dev), seq_ids=line, chunk=16)
    close(torch.cat([first[0], second[0, :26]]), ref, torch.float32, scale=5.0)
    assert float(second[0, 26:].abs().sum()) == 0.0
    for a, b in zip(st, st4):
        close(a[2], b[2].to("cpu", F64), torch.float32, scale=5.0)


@case
def test_head_norm_gate_squared_relu_and_norm_chain(dev, dt):
    torch.manual_seed(8)
    N, H, Dv = 7, 3, 10
    o = torch.randn(N, H, Dv) * 4
    src = torch.randn(N, 50).to(dt)
    w = torch.randn(H * Dv)
    y = ml.head_norm_gate(o.to(dev), src.to(dev), 11, H, Dv, w.to(dev), 1e-6, True, dt)
    ref = O.unit_rms(o.to(F64), 1e-6).reshape(N, H * Dv) * w.to(F64) * torch.sigmoid(src.to(F64)[:, 11:11 + H * Dv])
    close(y, ref, dt, scale=3.0)
    x = torch.randn(5, 33).to(dt)
    close(act_ops.relu_squared(x.to(dev)), torch.relu(x.to(F64)) ** 2, dt, scale=4.0)
    # post-norm + residual + next pre-norm on an fp32 stream with a large offset (the mean has to be removed)
    xs, yy = torch.randn(6, 70) * 20 + 300.0, (torch.randn(6, 70) * 3 + 50.0).to(dt)
    wp, wn = torch.randn(70), torch.randn(70)
    want_x = xs.to(F64) + O.layer_norm(yy.to(F64), wp.to(F64), 1e-6)
    got_x, hn = norm_ops.norm_chain_(xs.clone().to(dev), yy.to(dev), wp.to(dev), wn.to(dev), 1e-6, dt)
    assert got_x.dtype == torch.float32 and hn.dtype == dt
    close(got_x, want_x, torch.float32, scale=2.0)
    close(hn, O.layer_norm(want_x, wn.to(F64), 1e-6), dt, scale=3.0)
    _, first = norm_ops.norm_chain_(xs.clone().to(dev), None, None, wn.to(dev), 1e-6, dt)
    close(first, O.layer_norm(xs.to(F64), wn.to(F64), 1e-6), dt, scale=3.0)


def test_cache_holds_latent_rows_once_and_state_per_line():
    kc = KVCache(3, 2, 0, 16, 0, dtype=torch.float32, layer_specs=[(2, 4, 4), (1, 10, 8, "columns"), None],
                 state_specs={2: {"S": (2, 3, 5), "m": (2,)}})
    k, v = kc.layer(1)
    assert v.shape == (2, 1, 16, 8) and v.data_ptr() == k.data_ptr() and v.stride(2) == 10
    assert kc.layer(2) == (None, None) and kc.state(2)["S"].shape == (2, 2, 3, 5)
    assert kc.bytes() == 4 * (2 * 2 * 2 * 16 * 4 + 2 * 16 * 10 + 2 * (2 * 3 * 5 + 2))


def test_checkpoint_names_round_trip():
    cfg = tiny_rasodra()
    model = RasodraInferenceModel(cfg, InferenceConfig(batch_size=1, max_batch_size=1, seq_len=8, max_context_length=8))
    sd = export_rasodra_state_dict(model)
    back = convert_rasodra_state_dict(sd, cfg)
    ref = model.state_dict()
    assert set(back) == set(ref)
    for k in ref:
        assert torch.equal(back[k], ref[k]), k
    assert RasodraConfig.from_dict(cfg.to_dict(), torch.float32).to_dict() == cfg.to_dict()
    with pytest.raises(ValueError):
        RasodraConfig.from_dict(config(layers=[layer("attention"), layer("mlstm", weights_of=0)]))


# ---- the model through the framework -----------------------------------------------------------------------------------
@case
@pytest.mark.parametrize("cfg", [config(), ODD], ids=["mixed", "odd"])
def test_prefill_matches_oracle_and_token_by_token_decoding(dev, dt, cfg):
    toks = tokens_of(cfg, 45, 1)
    model, sd = build(cfg, dev, dt)
    streams = []
    ref = O.forward(cfg, sd, toks, streams)
    want = list(range(45))
    seen = []
    model.layer_probe = lambda i, x: seen.append(x.detach().to("cpu", F64))
    whole = replay(model, [([{"id": "a", "tokens": toks, "want": want}], ["a"])])["a"]
    model.layer_probe = None
    check_rows(whole, ref, want, dt)
    assert len(seen) == len(streams)
    for got, exp in zip(seen, streams):                       # the residual stream after every layer run
        assert float((got[0] - exp).abs().max()) <= (2e-3 if dt == torch.float32 else 0.5)
    steps = [([{"id": "b", "tokens": toks[:1], "want": [0]}], [])]
    steps += [([{"id": "b", "tokens": [t], "want": [0]}], []) for t in toks[1:]]
    check_rows(replay(model, steps)["b"], ref, want, dt)


@case
@pytest.mark.parametrize("portion", [2, 5, 16])
def test_portions_of_a_prompt(dev, dt, portion):
    cfg = config()
    toks = tokens_of(cfg, 41, 6)
    model, sd = build(cfg, dev, dt)
    ref = O.forward(cfg, sd, toks)
    steps, places = [], []
    for lo in range(0, 41, portion):
        part = toks[lo:lo + portion]
        steps.append(([{"id": "p", "tokens": part, "want": list(range(len(part)))}], []))
        places += list(range(lo, lo + len(part)))
    check_rows(replay(model, steps)["p"], ref, places, dt)


@case
def test_unequal_batch_equals_each_alone_and_lines_are_reused(dev, dt):
    cfg = config()
    model, sd = build(cfg, dev, dt, lines=3)
    lens = {"a": 1, "b": 30, "c": 13, "d": 22, "e": 9}
    toks = {k: tokens_of(cfg, n + 6, 10 + i) for i, (k, n) in enumerate(lens.items())}
    ref = {k: O.forward(cfg, sd, v) for k, v in toks.items()}
    first = [{"id": k, "tokens": toks[k][:lens[k]], "want": [lens[k] - 1]} for k in "abc"]
    steps = [(first, ["a"])]                                     # a one-token request ends at once: its line is free
    for s in range(3):
        steps.append(([{"id": k, "tokens": [toks[k][lens[k] + s]], "want": [0]} for k in "bc"], ["c"] if s == 2 else []))
    # two new requests take the lines that a and c gave back: stale keys and a stale recurrent state lie in them
    steps.append(([{"id": k, "tokens": toks[k][:lens[k]], "want": [0, lens[k] - 1]} for k in "de"], []))
    for s in range(6):
        steps.append(([{"id": k, "tokens": [toks[k][lens[k] + s]], "want": [0]} for k in "de"], []))
    got = replay(model, steps)
    check_rows(got["a"], ref["a"], [0], dt)
    for k in "bc":
        check_rows(got[k], ref[k], [lens[k] - 1, lens[k], lens[k] + 1, lens[k] + 2], dt)
    for k in "de":
        check_rows(got[k], ref[k], [0, lens[k] - 1] + [lens[k] + s for s in range(6)], dt)


@case
def test_long_prompt_steps_take_the_chunkwise_recurrence(dev, dt):
    """Steps of 64+ tokens run the recurrent layers in chunk-wise form (bf16 serving; forced here for fp32 too): a prompt
    of 150 tokens in two portions next to a short request, then decoding from the state they leave."""
    cfg = config(layers=[layer("mlstm", mlp=None), layer("mlstm"), layer("latent_attention", mlp=None)])
    model, sd = build(cfg, dev, dt, lines=2, seq_len=200)
    model.CHUNKWISE_FP32 = True
    a, b = tokens_of(cfg, 160, 31), tokens_of(cfg, 75, 32)
    ra, rb = O.forward(cfg, sd, a), O.forward(cfg, sd, b)
    steps = [([{"id": "a", "tokens": a[:80], "want": [0, 63, 64, 79]}, {"id": "b", "tokens": b[:70], "want": [69]}], []),
             ([{"id": "a", "tokens": a[80:150], "want": [0, 69]}], [])]
    steps += [([{"id": "a", "tokens": [a[150 + s]], "want": [0]}, {"id": "b", "tokens": [b[70 + s]], "want": [0]}], [])
              for s in range(5)]
    got = replay(model, steps)
    check_rows(got["a"], ra, [0, 63, 64, 79, 80, 149] + list(range(150, 155)), dt)
    check_rows(got["b"], rb, [69] + list(range(70, 75)), dt)


@case
def test_tensor_core_head_sizes_through_the_model(dev, dt):
    """Head sizes that the bf16 serving path runs on its tensor-core kernels: chunked attention with heads of 64 (prompts
    of a whole number of chunks run with the chunks as batch rows of the flash-attention kernel, other lengths and
    portions over the cache), latent attention with expanded heads of 96 | 64 and latent rows of 160 columns."""
    att = layer("attention", mlp=None, heads=2, kv_heads=1, dim=64, vdim=64, scale=0.125, mask={"size": 64},
                rot={"dims": 32, "base": 10000.0})
    lat = layer("latent_attention", mlp=None, heads=2, dim=64, rot_dim=32, vdim=64, kv_rank=128, scale=0.1,
                rot={"dims": 32, "base": 10000.0})
    cfg = config(layers=[att, lat, dict(att, weights_of=0)], width=64, vocab=80)
    model, sd = build(cfg, dev, dt, lines=3, seq_len=260)
    a, b, c = tokens_of(cfg, 200, 51), tokens_of(cfg, 140, 52), tokens_of(cfg, 230, 53)
    ra, rb, rc = (O.forward(cfg, sd, t) for t in (a, b, c))
    steps = [([{"id": "a", "tokens": a[:192], "want": [0, 63, 64, 127, 128, 191]},          # 3 chunks; b is padded to 192
               {"id": "b", "tokens": b[:130], "want": [64, 129]}], []),
             ([{"id": "c", "tokens": c[:150], "want": [149]}], []),                         # not a whole number of chunks
             ([{"id": "c", "tokens": c[150:220], "want": [0, 41, 42, 69]}], [])]            # a portion at an offset
    steps += [([{"id": "a", "tokens": [a[192 + s]], "want": [0]}, {"id": "b", "tokens": [b[130 + s]], "want": [0]},
                {"id": "c", "tokens": [c[220 + s]], "want": [0]}], []) for s in range(8)]
    got = replay(model, steps)
    check_rows(got["a"], ra, [0, 63, 64, 127, 128, 191] + list(range(192, 200)), dt)
    check_rows(got["b"], rb, [64, 129] + list(range(130, 138)), dt)
    check_rows(got["c"], rc, [149, 150, 191, 192, 219] + list(range(220, 228)), dt)


@case
def test_long_decoding_across_chunks_and_pages(dev, dt):
    cfg = config()
    toks = tokens_of(cfg, 90, 4)
    model, sd = build(cfg, dev, dt, lines=2, paged=True, pages=14, page_size=8)
    ref = O.forward(cfg, sd, toks)
    steps = [([{"id": "x", "tokens": toks[:5], "want": [4]}], [])]
    steps += [([{"id": "x", "tokens": [t], "want": [0]}], []) for t in toks[5:]]
    check_rows(replay(model, steps)["x"], ref, list(range(4, 90)), dt)


@case
def test_a_far_key_and_the_sink_decide_the_output(dev, dt):
    """One latent-attention layer whose inputs are normalised twice (layer norm, latent norm), so a key cannot be made
    to stand out by size alone.  Token id 5 sits at position 1 only and is the only token with a non-zero embedding
    column 1; one latent channel reads just that column, dimension 0 of every head's un-rotated key reads just that
    channel, and dimension 0 of every head's un-rotated query reads embedding column 0, which all tokens share.  So the
    key of position 1 takes the top score from every later query, hundreds of positions away, in the prompt and while
    decoding.  Then, on plain random weights, the sink of one head is raised until it takes most of that head's
    probability mass and another head's is removed: a run without sinks differs clearly."""
    cfg = config(layers=[layer("latent_attention", mlp=None)])
    m = cfg["layers"][0]["mixer"]
    H, D, R, C = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    base = O.random_weights(cfg, seed=3)
    sd = {k: v.clone() for k, v in base.items()}
    sd["embed"][:, 0] += 3.0
    sd["embed"][:, 1] = 0.0
    sd["embed"][5] = 0.0
    sd["embed"][5, 0], sd["embed"][5, 1] = 3.0, 8.0
    sd["l0.norm1"][0], sd["l0.norm1"][1] = 1.0, 1.0
    sd["l0.mix.dkv"][0] = 0.0
    sd["l0.mix.dkv"][0, 1] = 4.0
    sd["l0.mix.dkv.norm"][0] = 1.0
    for hd in range(H):
        sd["l0.mix.uk"][hd * D] = 0.0
        sd["l0.mix.uk"][hd * D, 0] = 1.0
        sd["l0.mix.q"][hd * (D + R)] = 0.0
        sd["l0.mix.q"][hd * (D + R), 0] = 8.0
    toks = [t if t != 5 else 6 for t in tokens_of(cfg, 300, 9)]
    toks[1] = 5
    sd = {k: v.to(torch.bfloat16).float() for k, v in sd.items()}
    model, _ = build(cfg, dev, dt, sd=sd, seq_len=320, lines=1)
    ref = O.forward(cfg, sd, toks)
    moved = list(toks)
    moved[1] = 6
    assert float((O.forward(cfg, sd, moved)[290] - ref[290]).abs().max()) > 0.05     # the far token matters
    steps = [([{"id": "f", "tokens": toks[:280], "want": [7, 8, 279]}], [])]
    steps += [([{"id": "f", "tokens": [t], "want": [0]}], []) for t in toks[280:]]
    check_rows(replay(model, steps)["f"], ref, [7, 8, 279] + list(range(280, 300)), dt)
    soft = config(layers=[layer("latent_attention", mlp=None, scale=0.02)])      # scores of order one: sinks weigh in
    sd2 = dict(base)
    sd2["l0.mix.sink"] = torch.tensor([3.0, -3.0, 0.5])     # the post-norm removes a scale common to all heads: differ
    none = dict(base)
    none["l0.mix.sink"] = torch.full((H,), -60.0)
    ref2 = O.forward(soft, sd2, toks[:40])
    assert float((ref2[30] - O.forward(soft, none, toks[:40])[30]).abs().max()) > 0.05
    model2, _ = build(soft, dev, dt, sd=sd2, lines=1)
    steps = [([{"id": "s", "tokens": toks[:33], "want": [0, 32]}], [])]
    steps += [([{"id": "s", "tokens": [t], "want": [0]}], []) for t in toks[33:40]]
    check_rows(replay(model2, steps)["s"], ref2, [0, 32] + list(range(33, 40)), dt)


@case
def test_chunk_edges_in_prompts_and_in_decoding(dev, dt):
    """One chunked-attention layer (chunk 8): the logits at the first and last position of a chunk, in a prompt that is
    cut inside a chunk and in decoding across the edge, equal the oracle's -- which differ from an oracle whose chunk is
    one position longer."""
    cfg = config(layers=[layer("attention", mlp=None)])
    sd = O.random_weights(cfg, seed=11)
    toks = tokens_of(cfg, 44, 2)
    ref = O.forward(cfg, sd, toks)
    other = config(layers=[layer("attention", mlp=None, mask={"size": 9})])
    assert float((O.forward(other, sd, toks)[16] - ref[16]).abs().max()) > 1e-3
    model, _ = build(cfg, dev, dt, sd=sd)
    steps = [([{"id": "c", "tokens": toks[:13], "want": [7, 8, 12]}], []),
             ([{"id": "c", "tokens": toks[13:30], "want": [2, 3, 10, 11, 16]}], [])]
    steps += [([{"id": "c", "tokens": [t], "want": [0]}], []) for t in toks[30:]]
    check_rows(replay(model, steps)["c"], ref, [7, 8, 12, 15, 16, 23, 24, 29] + list(range(30, 44)), dt)


@case
def test_greedy_generation_through_generate_and_the_continuous_batcher(dev, dt):
    cfg = config()
    sd = O.random_weights(cfg, seed=5)
    prompts = [tokens_of(cfg, n, 20 + n) for n in (7, 12, 3)]

    def oracle_greedy(p, new):
        seq = list(p)
        for _ in range(new):
            seq.append(int(O.forward(cfg, sd, seq)[-1].argmax()))
        return seq[len(p):]

    want = [oracle_greedy(p, 6) for p in prompts]
    model, _ = build(cfg, dev, dt, lines=3, sd=sd)
    T = max(len(p) for p in prompts)
    ids = torch.zeros(3, T, dtype=torch.long)
    mask = torch.zeros(3, T, dtype=torch.long)
    for b, p in enumerate(prompts):
        ids[b, :len(p)], mask[b, :len(p)] = torch.tensor(p), 1
    out = model.generate(ids.to(dev), mask.to(dev), max_new_tokens=6)
    strict = dt == torch.float32
    for b, p in enumerate(prompts):
        got = out[b, len(p):len(p) + 6].tolist()
        assert got == want[b] or not strict, (got, want[b])
        assert got[0] == want[b][0]
    # continuous batching over a page pool smaller than lines * pages per line: pages and lines (with their recurrent
    # state) are freed and handed out again
    from neuronx_distributed_llama3_2_b200.inference.continuous_batching import ContinuousBatcher

    model2, _ = build(cfg, dev, dt, lines=2, sd=sd, paged=True, pages=9, page_size=4, seq_len=32)
    cb = ContinuousBatcher(model2)
    rids = [cb.submit(torch.tensor(p), 6) for p in prompts]
    res = cb.run()
    for rid, w in zip(rids, want):
        assert res[rid][:6] == w or not strict, (res[rid], w)
        assert res[rid][0] == w[0]


@case
def test_runner_buckets_match_oracle_greedy(dev, dt):
    from neuronx_distributed_llama3_2_b200.inference import RasodraRunner

    cfg = config()
    sd = O.random_weights(cfg, seed=12)
    rc = RasodraConfig.from_dict(cfg, torch_dtype=dt)
    ic = InferenceConfig(batch_size=3, max_context_length=32, seq_len=64, buckets=[16, 32], max_new_tokens=5,
                         use_cuda_graphs=dev == "cuda")
    runner = RasodraRunner(rc, ic, checkpoint_loader=lambda: convert_rasodra_state_dict(sd, rc), device=torch.device(dev))
    runner.trace()
    prompts = [tokens_of(cfg, n, 40 + n) for n in (11, 5)]
    ids = torch.zeros(2, 11, dtype=torch.long)
    mask = torch.zeros(2, 11, dtype=torch.long)
    for b, p in enumerate(prompts):
        ids[b, :len(p)], mask[b, :len(p)] = torch.tensor(p), 1
    out = runner.generate(ids.to(dev), mask.to(dev), max_new_tokens=5)
    runner.close()
    for b, p in enumerate(prompts):
        seq = list(p)
        for _ in range(5):
            seq.append(int(O.forward(cfg, sd, seq)[-1].argmax()))
        got = out[b, len(p):len(p) + 5].tolist()
        assert got[0] == seq[len(p)]
        assert got == seq[len(p):] or dt != torch.float32, (got, seq[len(p):])


def test_registry_and_command_line_replay(tmp_path):
    """``bin/trace_run`` on a model directory: family chosen from config.json, steps on stdin, logits in files."""
    from safetensors.torch import save_file

    from neuronx_distributed_llama3_2_b200.inference.registry import families

    assert "rasodra" in families()
    cfg = ODD
    sd = O.random_weights(cfg, seed=8)
    mdir = tmp_path / "model"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in sd.items()}, str(mdir / "model.safetensors"))
    toks = tokens_of(cfg, 20, 3)
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:15], "want": [0, 14]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": toks[15:16], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "r", "tokens": toks[16:17], "want": [0]}], "end": ["r"]}]
    out = tmp_path / "out"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(mdir), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, env=env, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.split("\n") if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()
    ref = O.forward(cfg, sd, toks)
    import numpy as np

    a = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, cfg["vocab"]))
    b = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, cfg["vocab"]))
    check_rows([a[0], a[1], b[0]], ref, [0, 14, 16], torch.float32)
