"""Gekazen: a decoder-only family whose layers are listed one by one in the configuration.

Per layer: a mixer (``type``; ``attention`` is the one kind defined so far, others register in ``MIXERS``) and an
optional feed-forward.  What distinguishes the family from the Llama-shaped models of this package:

  * the residual stream ``x`` is fp32 and the norms sit on the sublayers' OUTPUTS: ``x += norm1(mixer(x))``,
    ``x += norm2(ff(x))``; norm weights are stored around zero (``1 + w``);
  * attention has biased projections, no rotation, queries and keys divided by their root mean square per head,
    a configured score scale, a linear distance bias with geometric per-head slopes, and a sliding window that keeps the
    first tokens visible; per-head key size and value size are independent; a layer may read another layer's keys and
    values (``kv_from``) instead of projecting its own;
  * the feed-forward is a sparse mixture (``modules/moe/sparse.py``): softmax router with a choice-only correction,
    scaled un-renormalised weights, identity experts, clamped gated activation, gated shared expert.

The configuration keys are the ones of the family's ``config.json``; checkpoints are converted by
``convert_gekazen_state_dict`` into this module's parameter names (fused q|k|v, stacked experts ``[E, in, out]``).
Tensor parallelism is not wired for this family (all layers are built for a tensor-parallel size of 1).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.nn as nn

from ..modules.moe import SparseMoE
from ..ops import window_attention as wa_ops
from ..parallel.layer_norm import ZeroCenteredRMSNorm
from ..parallel.layers import ColumnParallelLinear, ParallelEmbedding, RowParallelLinear

DISTANCE_SLOPE_EXPONENT = 8.0        # slope_h = 2 ** (-8 (h + 1) / heads)


@dataclass
class GekazenMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None       # mask.size; None = plain causal
    keep_first: int = 0                # mask.keep_first
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GekazenMixerConfig":
        mask = d.get("mask") or {}
        return cls(heads=int(d["heads"]), kv_heads=int(d.get("kv_heads", d["heads"])), dim=int(d["dim"]),
                   vdim=int(d.get("vdim", d["dim"])), scale=float(d["scale"]),
                   window=int(mask["size"]) if mask.get("size") is not None else None,
                   keep_first=int(mask.get("keep_first", 0) or 0),
                   kv_from=int(d["kv_from"]) if d.get("kv_from") is not None else None)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass
class GekazenMlpConfig:
    experts: int
    top: int
    ff: int
    limit: float
    identity: int = 0
    router_scale: float = 1.0
    shared_ff: int = 0
    shared_limit: Optional[float] = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GekazenMlpConfig":
        if d.get("kind", "moe") != "moe":
            raise ValueError(f"unknown feed-forward kind {d.get('kind')!r}")
        r, e, s = d["router"], d["expert"], d.get("shared")
        return cls(experts=int(r["experts"]), top=int(r["top"]), ff=int(e["ff"]), limit=float(e["limit"]),
                   identity=int(r.get("identity", 0) or 0), router_scale=float(r.get("scale", 1.0)),
                   shared_ff=int(s["ff"]) if s else 0, shared_limit=float(s["limit"]) if s else None)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
                             "router": {"experts": self.experts, "identity": self.identity, "scale": self.router_scale,
                                        "top": self.top}}
        d["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit} if self.shared_ff else None
        return d


@dataclass
class GekazenLayerConfig:
    type: str
    mixer: GekazenMixerConfig
    mlp: Optional[GekazenMlpConfig]


@dataclass
class GekazenConfig:
    vocab_size: int
    hidden_size: int
    layers: List[GekazenLayerConfig] = field(default_factory=list)
    rms_norm_eps: float = 1e-5
    torch_dtype: torch.dtype = torch.bfloat16
    model_type: str = "gekazen"
    # read by shared inference code
    sequence_parallel_enabled: bool = False
    activation_checkpointing: bool = False
    initializer_range: float = 0.02

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, d: Dict[str, Any], torch_dtype: torch.dtype = torch.bfloat16) -> "GekazenConfig":
        layers = []
        for i, L in enumerate(d["layers"]):
            if L["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r} (known: {sorted(MIXERS)})")
            mixer = GekazenMixerConfig.from_dict(L["mixer"])
            if mixer.kv_from is not None:
                src = d["layers"][mixer.kv_from]["mixer"] if 0 <= mixer.kv_from < i else None
                if src is None or src.get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier layer with projections of its own")
            layers.append(GekazenLayerConfig(L["type"], mixer, GekazenMlpConfig.from_dict(L["mlp"]) if L.get("mlp") else None))
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers,
                   rms_norm_eps=float(d["norm"]["eps"]), torch_dtype=torch_dtype)

    @classmethod
    def from_json(cls, path: str, torch_dtype: torch.dtype = torch.bfloat16) -> "GekazenConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f), torch_dtype)

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": "Gekazen", "vocab": self.vocab_size, "width": self.hidden_size,
                "norm": {"eps": self.rms_norm_eps},
                "layers": [{"type": L.type, "mixer": L.mixer.to_dict(), "mlp": L.mlp.to_dict() if L.mlp else None}
                           for L in self.layers]}


def _init(std: float) -> Callable:
    return lambda w: nn.init.normal_(w, mean=0.0, std=std)


class GekazenAttention(nn.Module):
    """Parameters and constants of the attention mixer; the forward over the KV cache lives in the inference model."""

    def __init__(self, config: GekazenConfig, mixer: GekazenMixerConfig, device=None):
        super().__init__()
        dt, W = config.torch_dtype, config.hidden_size
        self.cfg = mixer
        self.has_kv = mixer.kv_from is None
        n_out = mixer.heads * mixer.dim + (mixer.kv_heads * (mixer.dim + mixer.vdim) if self.has_kv else 0)
        init = _init(config.initializer_range)
        self.qkv_proj = ColumnParallelLinear(W, n_out, bias=True, gather_output=False, dtype=dt, device=device,
                                             init_method=init)
        self.o_proj = RowParallelLinear(mixer.heads * mixer.vdim, W, bias=True, input_is_parallel=True, dtype=dt,
                                        device=device, init_method=init)
        self.register_buffer("slopes", wa_ops.distance_slopes(mixer.heads, DISTANCE_SLOPE_EXPONENT, device=device),
                             persistent=False)


MIXERS: Dict[str, Callable[..., nn.Module]] = {"attention": GekazenAttention}


class GekazenDecoderLayer(nn.Module):
    def __init__(self, config: GekazenConfig, layer: GekazenLayerConfig, device=None):
        super().__init__()
        W, eps = config.hidden_size, config.rms_norm_eps
        self.type = layer.type
        self.self_attn = MIXERS[layer.type](config, layer.mixer, device=device)
        self.norm1 = ZeroCenteredRMSNorm(W, eps, device=device)
        self.mlp = None
        if layer.mlp is not None:
            m = layer.mlp
            self.mlp = SparseMoE(W, m.experts, m.top, m.ff, m.limit, num_identity_experts=m.identity,
                                 affinity_scale=m.router_scale, shared_intermediate_size=m.shared_ff,
                                 shared_limit=m.shared_limit, dtype=config.torch_dtype, device=device)
            self.norm2 = ZeroCenteredRMSNorm(W, eps, device=device)


class GekazenForCausalLM(nn.Module):
    def __init__(self, config: GekazenConfig, device=None):
        super().__init__()
        self.config = config
        dt = config.torch_dtype
        self.embed_tokens = ParallelEmbedding(config.vocab_size, config.hidden_size, dtype=dt, device=device,
                                              init_method=_init(config.initializer_range))
        self.layers = nn.ModuleList([GekazenDecoderLayer(config, L, device=device) for L in config.layers])
        self.norm = ZeroCenteredRMSNorm(config.hidden_size, config.rms_norm_eps, device=device)
        self.lm_head = ColumnParallelLinear(config.hidden_size, config.vocab_size, bias=False, gather_output=False,
                                            dtype=dt, device=device, init_method=_init(config.initializer_range))


def convert_gekazen_state_dict(sd: Dict[str, torch.Tensor], config: GekazenConfig) -> Dict[str, torch.Tensor]:
    """Checkpoint names (``embed``, ``l<i>.mix.q`` / ``.q.b``, ``l<i>.mlp.e<j>.gate`` ..., ``final.norm``, ``head``;
    linear weights ``[out, in]``) -> this module's state dict."""
    out: Dict[str, torch.Tensor] = {"embed_tokens.weight": sd["embed"], "lm_head.weight": sd["head"],
                                    "norm.weight": sd["final.norm"].float()}
    for i, L in enumerate(config.layers):
        src, dst = f"l{i}.", f"layers.{i}."
        names = ["q"] + (["k", "v"] if L.mixer.kv_from is None else [])
        out[dst + "self_attn.qkv_proj.weight"] = torch.cat([sd[src + "mix." + n] for n in names], dim=0)
        out[dst + "self_attn.qkv_proj.bias"] = torch.cat([sd[src + "mix." + n + ".b"] for n in names], dim=0)
        out[dst + "self_attn.o_proj.weight"] = sd[src + "mix.o"]
        out[dst + "self_attn.o_proj.bias"] = sd[src + "mix.o.b"]
        out[dst + "norm1.weight"] = sd[src + "norm1"].float()
        if L.mlp is None:
            continue
        m = L.mlp
        out[dst + "norm2.weight"] = sd[src + "norm2"].float()
        out[dst + "mlp.router.linear_router.weight"] = sd[src + "mlp.router"].float()
        out[dst + "mlp.router.correction"] = sd[src + "mlp.correction"].float()
        out[dst + "mlp.experts.gate_up_proj.weight"] = torch.stack(
            [torch.cat([sd[f"{src}mlp.e{e}.gate"].t(), sd[f"{src}mlp.e{e}.up"].t()], dim=1) for e in range(m.experts)])
        out[dst + "mlp.experts.down_proj.weight"] = torch.stack([sd[f"{src}mlp.e{e}.down"].t() for e in range(m.experts)])
        if m.shared_ff:
            out[dst + "mlp.shared.gate_up_proj.weight"] = torch.cat(
                [sd[src + "mlp.shared.gate"].t(), sd[src + "mlp.shared.up"].t()], dim=1).unsqueeze(0)
            out[dst + "mlp.shared.down_proj.weight"] = sd[src + "mlp.shared.down"].t().unsqueeze(0)
            out[dst + "mlp.shared_gate.weight"] = sd[src + "mlp.shared.sg"].float().reshape(1, -1)
    return {k: v.contiguous() for k, v in out.items()}


def tiny_gekazen(torch_dtype: torch.dtype = torch.float32, **kw) -> GekazenConfig:
    """A small configuration for tests and smoke runs: four layers, grouped key/value heads, key size != value size,
    one layer without a feed-forward, one layer that reads another layer's keys and values."""
    def mixer(**m):
        base = dict(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.2, mask={"size": 12, "keep_first": 3})
        base.update(m)
        return base

    def mlp(**m):
        base = {"kind": "moe", "expert": {"ff": 32, "limit": 2.0},
                "router": {"experts": 6, "identity": 1, "scale": 1.25, "top": 2}, "shared": {"ff": 40, "limit": 1.5}}
        base.update(m)
        return base

    d = {"architecture": "Gekazen", "vocab": 160, "width": 48, "norm": {"eps": 1e-5},
         "layers": [{"type": "attention", "mixer": mixer(), "mlp": mlp()},
                    {"type": "attention", "mixer": mixer(mask={"size": 7, "keep_first": 0}), "mlp": None},
                    {"type": "attention", "mixer": mixer(kv_from=0, mask={"size": 20, "keep_first": 2}), "mlp": mlp(shared=None)},
                    {"type": "attention", "mixer": mixer(heads=2, kv_heads=2, dim=24, vdim=16), "mlp": mlp()}]}
    d.update(kw)
    return GekazenConfig.from_dict(d, torch_dtype=torch_dtype)
