"""Latent (compressed key/value) attention: the step's work on the fused projection output before the attention kernel
(``csrc/latent_attention.cu``).

The projection row of a token holds ``heads`` query heads laid out ``[dim un-rotated | rot rotated]`` and ``rank``
compressed key/value columns followed by ``rot`` columns of one rotated key part shared by all heads.  The cache keeps
one row per token, ``[c | k_rot]`` with ``c = rms_norm(compressed) * weight``.  Because

    score_h(i, j) = <q_nope_h, W_uk_h c_j> + <q_rot_h, k_rot_j> = <[W_uk_h^T q_nope_h | q_rot_h], [c_j | k_rot_j]>

all heads attend to the same rows with an absorbed query (``ops.window_attention`` with one key/value head whose value
is the ``c`` part of the row), and the per-head value projection follows the attention.
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional, Tuple

import torch

from . import _lib
from .rope import rope_interleaved_ref

GROUP = "hybrid_serving"


def _i32(t):
    if t is None:
        return None
    return t if (t.dtype == torch.int32 and t.is_contiguous()) else t.to(torch.int32).contiguous()


def latent_prep(proj: torch.Tensor, q_off: int, kv_off: int, q_abs: Optional[torch.Tensor], cache: torch.Tensor,
                c_weight: torch.Tensor, rope: Tuple[torch.Tensor, torch.Tensor], q_start: torch.Tensor, heads: int,
                dim: int, rot: int, rank: int, eps: float, n_new: Optional[torch.Tensor] = None,
                seq_ids: Optional[torch.Tensor] = None, block_table: Optional[torch.Tensor] = None,
                page_size: int = 0) -> torch.Tensor:
    """``proj [B, T, ld]``.  Writes the cache row ``[c | k_rot]`` of every real token at (line, position);
    ``cache [lines | pages, 1, rows, rank + rot]``.  With ``q_abs [B*T, heads, rank + rot]`` (token generation): returns
    ``q_nope [B*T, heads, dim]`` (the un-rotated query columns, for the absorption product) and fills
    ``q_abs[..., rank:]`` with the rotated query part.  With ``q_abs=None`` (prompt steps): returns the queries
    ``[B*T, heads, dim + rot]`` with their rotated part turned."""
    B, T, ld = proj.shape
    N = B * T
    cos, sin = rope
    if q_abs is None:
        q_full = torch.empty(N, heads, dim + rot, dtype=proj.dtype, device=proj.device)
        q_nope, nope_head, q_rot, rot_head, ret = q_full, dim + rot, q_full[..., dim:], dim + rot, q_full
    else:
        q_nope = torch.empty(N, heads, dim, dtype=proj.dtype, device=proj.device)
        nope_head, q_rot, rot_head, ret = dim, q_abs[..., rank:], rank + rot, q_nope
    if proj.is_cuda and proj.dtype in (torch.bfloat16, torch.float32) and _lib.available(GROUP):
        assert proj.is_contiguous() and (q_abs is None or q_abs.is_contiguous()) and cache.stride(3) == 1
        bt, qs, nn_, sid = _i32(block_table), _i32(q_start), _i32(n_new), _i32(seq_ids)   # alive across the launch
        max_pos = bt.shape[1] * page_size if bt is not None else cache.shape[2]
        L = _lib.lib(GROUP)
        rc = L.nxd_latent_prep(_c.c_int({torch.bfloat16: 0, torch.float32: 1}[proj.dtype]), _lib.ptr(proj),
                               _c.c_longlong(ld), _c.c_int(q_off), _c.c_int(kv_off), _lib.ptr(q_nope),
                               _c.c_longlong(nope_head), _c.c_void_p(q_rot.data_ptr()), _c.c_longlong(rot_head),
                               _lib.ptr(cache),
                               _c.c_longlong(cache.stride(0)), _c.c_longlong(cache.stride(2)), _lib.ptr(bt),
                               _c.c_int(page_size if bt is not None else 0), _c.c_int(bt.shape[1] if bt is not None else 0),
                               _lib.ptr(c_weight), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(qs),
                               _lib.ptr(nn_), _lib.ptr(sid), _c.c_int(B), _c.c_int(T), _c.c_int(heads),
                               _c.c_int(dim), _c.c_int(rot), _c.c_int(rank), _c.c_float(eps), _c.c_int(max_pos),
                               _lib.stream_ptr())
        _lib.check(rc, "nxd_latent_prep", L)
        return ret
    pos = q_start.long().reshape(B, 1) + torch.arange(T, device=proj.device).reshape(1, T)
    q = proj[..., q_off: q_off + heads * (dim + rot)].reshape(B, T, heads, dim + rot)
    q_nope[..., :dim] = q[..., :dim].reshape(N, heads, dim)
    q_rot.copy_(rope_interleaved_ref(q[..., dim:].float(), pos, cos, sin).to(proj.dtype).reshape(N, heads, rot))
    kv = proj[..., kv_off: kv_off + rank + rot].float()
    c = kv[..., :rank]
    c = c / torch.sqrt(c.pow(2).mean(-1, keepdim=True) + eps) * c_weight.float()
    kr = rope_interleaved_ref(kv[..., rank:].unsqueeze(-2), pos, cos, sin).squeeze(-2)
    rows = torch.cat([c, kr], dim=-1).to(cache.dtype)
    for b in range(B):
        cnt = T if n_new is None else min(int(n_new[b]), T)
        line = b if seq_ids is None else int(seq_ids[b])
        for t in range(cnt):
            p = int(q_start[b]) + t
            if block_table is not None:
                cache[int(block_table[line, p // page_size]), 0, p % page_size] = rows[b, t]
            else:
                cache[line, 0, p] = rows[b, t]
    return ret


TARGET_CTAS = 296          # two CTAs' worth of work per SM before the context is split further


def latent_decode(q_abs: torch.Tensor, cache: torch.Tensor, value_cols: int, out: torch.Tensor, positions: torch.Tensor,
                  seq_ids: Optional[torch.Tensor], sinks: Optional[torch.Tensor], scale: float,
                  block_table: Optional[torch.Tensor], page_size: int) -> bool:
    """Token generation over latent rows on tensor cores (``csrc/latent_attention.cu: latent_decode_kernel``):
    ``q_abs [B, H, D]`` bf16 absorbed queries, ``cache [lines | pages, 1, rows, D]`` whose first ``value_cols`` columns
    are the values, ``positions`` / ``seq_ids`` / ``block_table`` int32, ``sinks`` fp32.  Fills ``out [B, H, value_cols]``
    and returns True; returns False when no kernel is compiled for these sizes (the caller takes the general kernels)."""
    B, H, D = q_abs.shape
    rows = block_table.shape[1] * page_size if block_table is not None else cache.shape[2]
    ctas = ((H + 15) // 16) * B
    nsplit = max(1, min(8, TARGET_CTAS // max(ctas, 1), (rows + 63) // 64))
    partial = (torch.empty(B, H, nsplit, value_cols + 2, dtype=torch.float32, device=q_abs.device) if nsplit > 1 else None)
    L = _lib.lib(GROUP)
    rc = L.nxd_latent_decode(_lib.ptr(q_abs), _lib.ptr(cache), _c.c_longlong(cache.stride(0)),
                             _c.c_longlong(cache.stride(2)), _lib.ptr(block_table),
                             _c.c_int(page_size if block_table is not None else 0),
                             _c.c_int(block_table.shape[1] if block_table is not None else 0), _lib.ptr(out),
                             _lib.ptr(partial), _lib.ptr(positions), _lib.ptr(seq_ids), _lib.ptr(sinks), _c.c_int(B),
                             _c.c_int(H), _c.c_int(D), _c.c_int(value_cols), _c.c_float(scale), _c.c_int(nsplit),
                             _lib.stream_ptr())
    if rc == 2:
        return False
    _lib.check(rc, "nxd_latent_decode", L)
    return True
