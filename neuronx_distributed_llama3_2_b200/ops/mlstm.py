"""Matrix-memory recurrent mixer (mLSTM) ops over a per-line fp32 state (``csrc/mlstm.cu``), and the gated head output
that follows it.

Per head, with log-space input / forget gates ``i_t`` / ``f_t`` and a running maximum ``m`` (``m_0 = 0``, zero state):

    m_t = max(f_t + m_{t-1}, i_t)
    S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T
    n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)

Gates, state and the division are fp32 whatever the activation dtype.  A row whose first position is 0 starts from the
zero state; any other row continues from the state its cache line holds, so a prompt may arrive in portions and a line
that is handed to a new request needs no clearing.  Every op has a PyTorch restatement for CPU.
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib

GROUP = "hybrid_serving"
DENOMINATOR_FLOOR = 1e-6


def _code(dtype: torch.dtype) -> int:
    return {torch.bfloat16: 0, torch.float32: 1}[dtype]


def _use_kernel(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and _lib.available(GROUP)


def _i32(t):
    if t is None:
        return None
    return t if (t.dtype == torch.int32 and t.is_contiguous()) else t.to(torch.int32).contiguous()


def soft_cap(x: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(x / cap) if cap and cap > 0 else x


def mlstm_gates(h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor, heads: int, cap: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """``h [N, W]``, ``w [2 * heads, W]`` (input-gate rows, then forget-gate rows), ``bias [2 * heads]`` fp32 ->
    fp32 ``(i, f) [N, heads]``: ``i = cap tanh(x_i / cap)``, ``f = logsigmoid(cap tanh(x_f / cap))``.  The dot
    products accumulate in fp32 and are never rounded to the activation dtype."""
    N, W = h.shape
    if _use_kernel(h) and w.dtype == h.dtype:
        h2 = h if h.is_contiguous() else h.contiguous()
        gi = torch.empty(N, heads, dtype=torch.float32, device=h.device)
        gf = torch.empty(N, heads, dtype=torch.float32, device=h.device)
        L = _lib.lib(GROUP)
        rc = L.nxd_mlstm_gates(_c.c_int(_code(h.dtype)), _lib.ptr(h2), _lib.ptr(w), _lib.ptr(bias), _lib.ptr(gi),
                               _lib.ptr(gf), _c.c_longlong(N), _c.c_int(W), _c.c_int(heads), _c.c_float(cap),
                               _lib.stream_ptr())
        _lib.check(rc, "nxd_mlstm_gates", L)
        return gi, gf
    pre = h.float() @ w.float().t() + bias.float()
    return soft_cap(pre[:, :heads], cap), F.logsigmoid(soft_cap(pre[:, heads:], cap))


def mlstm_scan(proj: torch.Tensor, offsets: Tuple[int, int, int], gi: torch.Tensor, gf: torch.Tensor,
               state: Tuple[torch.Tensor, torch.Tensor, torch.Tensor], q_start: torch.Tensor, heads: int, dim: int,
               vdim: int, qscale: float, n_new: Optional[torch.Tensor] = None,
               seq_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``proj [B, T, ld]`` holds the step's queries / keys / values head-major at column ``offsets = (q, k, v)``;
    ``gi / gf [B * T, heads]`` fp32; ``state = (S [lines, heads, dim, vdim], n [lines, heads, dim], m [lines, heads])``
    fp32, updated in place for line ``seq_ids[b]`` (default ``b``).  Tokens ``t >= n_new[b]`` are padding: they leave
    the state alone and come out as zeros.  Returns fp32 ``o [B, T, heads, vdim]``."""
    B, T, ld = proj.shape
    S, n, m = state
    if _use_kernel(proj):
        assert proj.is_contiguous() and S.is_contiguous() and n.is_contiguous() and m.is_contiguous()
        out = torch.empty(B, T, heads, vdim, dtype=torch.float32, device=proj.device)
        nxn = torch.empty(B, heads, dim, dtype=torch.float32, device=proj.device)
        nxm = torch.empty(B, heads, dtype=torch.float32, device=proj.device)
        qs, nn_, sid = _i32(q_start), _i32(n_new), _i32(seq_ids)      # converted copies stay alive across the launch
        L = _lib.lib(GROUP)
        rc = L.nxd_mlstm_scan(_c.c_int(_code(proj.dtype)), _lib.ptr(proj), _c.c_longlong(ld), _c.c_int(offsets[0]),
                              _c.c_int(offsets[1]), _c.c_int(offsets[2]), _lib.ptr(gi), _lib.ptr(gf), _lib.ptr(S),
                              _lib.ptr(n), _lib.ptr(m), _lib.ptr(nxn), _lib.ptr(nxm), _lib.ptr(out), _lib.ptr(qs),
                              _lib.ptr(nn_), _lib.ptr(sid), _c.c_int(B), _c.c_int(T), _c.c_int(heads),
                              _c.c_int(dim), _c.c_int(vdim), _c.c_float(qscale), _lib.stream_ptr())
        _lib.check(rc, "nxd_mlstm_scan", L)
        return out
    out = torch.zeros(B, T, heads, vdim, dtype=torch.float32, device=proj.device)
    q = proj[..., offsets[0]: offsets[0] + heads * dim].float().reshape(B, T, heads, dim) * qscale
    k = proj[..., offsets[1]: offsets[1] + heads * dim].float().reshape(B, T, heads, dim)
    v = proj[..., offsets[2]: offsets[2] + heads * vdim].float().reshape(B, T, heads, vdim)
    gi, gf = gi.reshape(B, T, heads), gf.reshape(B, T, heads)
    for b in range(B):
        cnt = T if n_new is None else min(int(n_new[b]), T)
        if cnt <= 0:
            continue
        line = b if seq_ids is None else int(seq_ids[b])
        if int(q_start[b]) == 0:
            Sb, nb, mb = torch.zeros_like(S[line]), torch.zeros_like(n[line]), torch.zeros_like(m[line])
        else:
            Sb, nb, mb = S[line].clone(), n[line].clone(), m[line].clone()
        for t in range(cnt):
            mn = torch.maximum(gf[b, t] + mb, gi[b, t])
            a, w = torch.exp(gf[b, t] + mb - mn), torch.exp(gi[b, t] - mn)
            Sb = a[:, None, None] * Sb + (w[:, None] * k[b, t])[:, :, None] * v[b, t][:, None, :]
            nb = a[:, None] * nb + w[:, None] * k[b, t]
            mb = mn
            den = torch.maximum((nb * q[b, t]).sum(-1).abs(), torch.exp(-mb)) + DENOMINATOR_FLOOR
            out[b, t] = torch.einsum("hdv,hd->hv", Sb, q[b, t]) / den[:, None]
        S[line], n[line], m[line] = Sb, nb, mb
    return out


def head_norm_gate(o: torch.Tensor, gate_src: torch.Tensor, gate_offset: int, heads: int, vdim: int,
                   weight: Optional[torch.Tensor], eps: float, normalize: bool, out_dtype: torch.dtype) -> torch.Tensor:
    """``o [N, heads, vdim]`` -> ``[N, heads * vdim]`` in ``out_dtype``: every head divided by its root mean square
    (``normalize``; fp32, ``eps`` inside the root), times ``weight [heads * vdim]`` (optional), times
    ``sigmoid(gate)`` where the gate pre-activations are columns ``gate_offset ...`` of ``gate_src [N, ld]``."""
    N = o.shape[0]
    ld = gate_src.shape[-1]
    if (_use_kernel(gate_src) and gate_src.dtype == out_dtype and gate_src.is_contiguous() and o.is_contiguous()
            and (o.dtype == torch.float32 or o.dtype == out_dtype)):
        out = torch.empty(N, heads * vdim, dtype=out_dtype, device=o.device)
        wf = weight.float().contiguous() if weight is not None else None
        L = _lib.lib(GROUP)
        rc = L.nxd_head_norm_gate(_c.c_int(_code(o.dtype)), _c.c_int(_code(out_dtype)), _lib.ptr(o), _lib.ptr(gate_src),
                                  _c.c_longlong(ld), _c.c_int(gate_offset), _lib.ptr(wf), _lib.ptr(out), _c.c_longlong(N),
                                  _c.c_int(heads), _c.c_int(vdim), _c.c_int(int(normalize)), _c.c_float(eps),
                                  _lib.stream_ptr())
        _lib.check(rc, "nxd_head_norm_gate", L)
        return out
    of = o.float().reshape(N, heads, vdim)
    if normalize:
        of = of / torch.sqrt(of.pow(2).mean(-1, keepdim=True) + eps)
    of = of.reshape(N, heads * vdim)
    if weight is not None:
        of = of * weight.float()
    g = gate_src.reshape(N, ld)[:, gate_offset: gate_offset + heads * vdim].float()
    return (of * torch.sigmoid(g)).to(out_dtype)
