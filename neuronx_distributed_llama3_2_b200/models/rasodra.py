"""Rasodra: a decoder-only hybrid family.  The configuration lists the layers one by one; each has a mixer of one of
three kinds and an optional dense feed-forward, and a layer may run with the weights of an earlier layer.

  * the residual stream ``x`` is fp32, with a weight-only layer norm BEFORE and AFTER every sublayer:
    ``x += norm1b(mixer(norm1(x)))``, ``x += norm2b(ff(norm2(x)))``;
  * ``attention``: grouped-query attention whose values are the raw key projections (there is no value matrix), biased q / k
    projections, per-head RMS norm of q and k with a shared weight, interleaved rotary positions on the first
    ``rot.dims`` dimensions, a configured score scale and a CHUNKED causal mask (a query sees the keys of its own chunk
    of ``mask.size`` positions, chunk boundaries at absolute multiples of the size);
  * ``latent_attention``: keys and values are up-projections of a small normalised latent ``c`` per token, plus one
    rotated key part shared by all heads; only ``c`` and that part are cached.  Softmax with a learned per-head sink
    logit in the denominator, sigmoid output gate;
  * ``mlstm``: a matrix memory per head, updated token by token with exponential input / sigmoid forget gates kept
    stable by a running maximum (xLSTM's mLSTM; Beck et al., "xLSTM: Extended Long Short-Term Memory"), soft-capped
    gate pre-activations, per-head unit-RMS output norm and sigmoid output gate;
  * feed-forward: ``down(relu(up(h)) ** 2)``;
  * ``weights_of: j`` on a layer: it has no tensors of its own and runs with layer ``j``'s modules, on a cache / state
    of its own.

Parameter modules only; the forward over the KV cache and the recurrent state lives in
``inference/hybrid.py: RasodraInferenceModel``.  Tensor parallelism is not wired for this family.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.nn as nn

from ..parallel.layer_norm import WeightOnlyLayerNorm
from ..parallel.layers import ColumnParallelLinear, ParallelEmbedding, RowParallelLinear


@dataclass
class RotaryConfig:
    dims: int
    base: float

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> Optional["RotaryConfig"]:
        return cls(dims=int(d["dims"]), base=float(d["base"])) if d else None

    def to_dict(self) -> Dict[str, Any]:
        return {"dims": self.dims, "base": self.base}


@dataclass
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int]               # mask.size; None = plain causal
    rot: Optional[RotaryConfig]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ChunkedAttentionConfig":
        mask = d.get("mask") or {}
        c = cls(heads=int(d["heads"]), kv_heads=int(d.get("kv_heads", d["heads"])), dim=int(d["dim"]),
                vdim=int(d.get("vdim", d["dim"])), scale=float(d["scale"]),
                chunk=int(mask["size"]) if mask.get("size") else None, rot=RotaryConfig.from_dict(d.get("rot")))
        if c.vdim != c.dim:
            raise ValueError(f"attention: the values are the projected keys, so vdim ({c.vdim}) must equal dim ({c.dim})")
        if c.heads % c.kv_heads:
            raise ValueError(f"attention: {c.heads} query heads over {c.kv_heads} key/value heads")
        if c.rot is not None and (c.rot.dims % 2 or c.rot.dims > c.dim):
            raise ValueError(f"attention: rotation over {c.rot.dims} of {c.dim} dimensions")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.chunk:
            d["mask"] = {"size": self.chunk}
        if self.rot:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass
class LatentAttentionConfig:
    heads: int
    dim: int                           # un-rotated query / key dimensions per head
    rot_dim: int                       # rotated dimensions per head (the key's are shared by all heads)
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LatentAttentionConfig":
        c = cls(heads=int(d["heads"]), dim=int(d["dim"]), rot_dim=int(d["rot_dim"]), vdim=int(d["vdim"]),
                kv_rank=int(d["kv_rank"]), scale=float(d["scale"]), rot=RotaryConfig.from_dict(d["rot"]))
        if c.rot.dims != c.rot_dim or c.rot_dim % 2:
            raise ValueError(f"latent attention: rot.dims ({c.rot.dims}) must equal rot_dim ({c.rot_dim}), an even number")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "scale": self.scale, "rot": self.rot.to_dict()}


@dataclass
class MLstmConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MLstmConfig":
        return cls(heads=int(d["heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]), gate_cap=float(d["gate_cap"]))

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass
class DenseMlpConfig:
    ff: int

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DenseMlpConfig":
        if d.get("kind", "dense") != "dense":
            raise ValueError(f"unknown feed-forward kind {d.get('kind')!r}")
        return cls(ff=int(d["ff"]))

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


MIXER_CONFIGS: Dict[str, Any] = {"attention": ChunkedAttentionConfig, "latent_attention": LatentAttentionConfig,
                                 "mlstm": MLstmConfig}


@dataclass
class RasodraLayerConfig:
    type: str
    mixer: Any
    mlp: Optional[DenseMlpConfig]
    weights_of: Optional[int] = None


@dataclass
class RasodraConfig:
    vocab_size: int
    hidden_size: int
    layers: List[RasodraLayerConfig] = field(default_factory=list)
    rms_norm_eps: float = 1e-6
    torch_dtype: torch.dtype = torch.bfloat16
    model_type: str = "rasodra"
    # read by shared inference code
    sequence_parallel_enabled: bool = False
    activation_checkpointing: bool = False
    initializer_range: float = 0.02

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def owner(self, i: int) -> int:
        """Index of the layer whose modules layer ``i`` runs with."""
        j = self.layers[i].weights_of
        return i if j is None else j

    @classmethod
    def from_dict(cls, d: Dict[str, Any], torch_dtype: torch.dtype = torch.bfloat16) -> "RasodraConfig":
        layers: List[RasodraLayerConfig] = []
        for i, L in enumerate(d["layers"]):
            if L["type"] not in MIXER_CONFIGS:
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r} (known: {sorted(MIXER_CONFIGS)})")
            j = L.get("weights_of")
            if j is not None:
                j = int(j)
                if not (0 <= j < i) or d["layers"][j].get("weights_of") is not None or d["layers"][j]["type"] != L["type"]:
                    raise ValueError(f"layer {i}: weights_of must name an earlier layer of the same type with tensors of its own")
            layers.append(RasodraLayerConfig(L["type"], MIXER_CONFIGS[L["type"]].from_dict(L["mixer"]),
                                             DenseMlpConfig.from_dict(L["mlp"]) if L.get("mlp") else None, j))
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers,
                   rms_norm_eps=float(d["norm"]["eps"]), torch_dtype=torch_dtype)

    @classmethod
    def from_json(cls, path: str, torch_dtype: torch.dtype = torch.bfloat16) -> "RasodraConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f), torch_dtype)

    def to_dict(self) -> Dict[str, Any]:
        out = []
        for L in self.layers:
            e: Dict[str, Any] = {"type": L.type, "mixer": L.mixer.to_dict(), "mlp": L.mlp.to_dict() if L.mlp else None}
            if L.weights_of is not None:
                e["weights_of"] = L.weights_of
            out.append(e)
        return {"architecture": "Rasodra", "vocab": self.vocab_size, "width": self.hidden_size,
                "norm": {"eps": self.rms_norm_eps}, "layers": out}


def _init(std: float) -> Callable:
    return lambda w: nn.init.normal_(w, mean=0.0, std=std)


def _linear_in(config: RasodraConfig, n_out: int, bias: bool, device) -> ColumnParallelLinear:
    return ColumnParallelLinear(config.hidden_size, n_out, bias=bias, gather_output=False, dtype=config.torch_dtype,
                                device=device, init_method=_init(config.initializer_range))


def _linear_out(config: RasodraConfig, n_in: int, device) -> RowParallelLinear:
    return RowParallelLinear(n_in, config.hidden_size, bias=False, input_is_parallel=True, dtype=config.torch_dtype,
                             device=device, init_method=_init(config.initializer_range))


class ChunkedAttentionMixer(nn.Module):
    """q | k in one biased projection (the raw key projections double as values), norm weights of q and k, output
    projection."""

    def __init__(self, config: RasodraConfig, m: ChunkedAttentionConfig, device=None):
        super().__init__()
        self.cfg = m
        self.qk_proj = _linear_in(config, (m.heads + m.kv_heads) * m.dim, True, device)
        self.q_norm = nn.Parameter(torch.ones(m.dim, dtype=torch.float32, device=device))
        self.k_norm = nn.Parameter(torch.ones(m.dim, dtype=torch.float32, device=device))
        self.o_proj = _linear_out(config, m.heads * m.vdim, device)


class LatentAttentionMixer(nn.Module):
    """q | compressed kv (+ shared rotated key part) | output gate in one projection; latent norm weight; per-head
    up-projections kept per head, ``uk [heads, dim, rank]`` and ``uv [heads, vdim, rank]``: token generation absorbs
    ``uk`` into the query and applies ``uv`` to the attention output over the latent rows; prompt steps expand keys and
    values from the latent rows with the same two tensors viewed as ``[heads * dim, rank]`` / ``[heads * vdim, rank]``;
    sink logits; output projection."""

    def __init__(self, config: RasodraConfig, m: LatentAttentionConfig, device=None):
        super().__init__()
        self.cfg = m
        dt, std = config.torch_dtype, config.initializer_range
        self.q_cols = m.heads * (m.dim + m.rot_dim)
        self.kv_cols = m.kv_rank + m.rot_dim
        self.in_proj = _linear_in(config, self.q_cols + self.kv_cols + m.heads * m.vdim, False, device)
        self.kv_norm = nn.Parameter(torch.ones(m.kv_rank, dtype=torch.float32, device=device))
        self.uk = nn.Parameter(torch.empty(m.heads, m.dim, m.kv_rank, dtype=dt, device=device).normal_(0.0, std))
        self.uv = nn.Parameter(torch.empty(m.heads, m.vdim, m.kv_rank, dtype=dt, device=device).normal_(0.0, std))
        self.sink = nn.Parameter(torch.zeros(m.heads, dtype=torch.float32, device=device))
        self.o_proj = _linear_out(config, m.heads * m.vdim, device)


class MLstmMixer(nn.Module):
    """q | k | v | output gate in one projection; the two gate rows per head stay separate (``gate_weight [2 * heads,
    width]``: input gates, then forget gates) because their dot products are kept in fp32; per-head output norm weight;
    output projection."""

    def __init__(self, config: RasodraConfig, m: MLstmConfig, device=None):
        super().__init__()
        self.cfg = m
        dt, std = config.torch_dtype, config.initializer_range
        self.in_proj = _linear_in(config, 2 * m.heads * m.dim + 2 * m.heads * m.vdim, False, device)
        self.gate_weight = nn.Parameter(torch.empty(2 * m.heads, config.hidden_size, dtype=dt, device=device).normal_(0.0, std))
        self.gate_bias = nn.Parameter(torch.zeros(2 * m.heads, dtype=torch.float32, device=device))
        self.out_norm = nn.Parameter(torch.ones(m.heads * m.vdim, dtype=torch.float32, device=device))
        self.o_proj = _linear_out(config, m.heads * m.vdim, device)


MIXERS: Dict[str, Callable[..., nn.Module]] = {"attention": ChunkedAttentionMixer,
                                               "latent_attention": LatentAttentionMixer, "mlstm": MLstmMixer}


class DenseMlp(nn.Module):
    def __init__(self, config: RasodraConfig, m: DenseMlpConfig, device=None):
        super().__init__()
        self.up_proj = _linear_in(config, m.ff, False, device)
        self.down_proj = _linear_out(config, m.ff, device)


class RasodraDecoderLayer(nn.Module):
    def __init__(self, config: RasodraConfig, layer: RasodraLayerConfig, device=None):
        super().__init__()
        W, eps = config.hidden_size, config.rms_norm_eps
        self.type = layer.type
        self.mixer = MIXERS[layer.type](config, layer.mixer, device=device)
        self.norm1 = WeightOnlyLayerNorm(W, eps, device=device)
        self.norm1b = WeightOnlyLayerNorm(W, eps, device=device)
        self.mlp = None
        if layer.mlp is not None:
            self.mlp = DenseMlp(config, layer.mlp, device=device)
            self.norm2 = WeightOnlyLayerNorm(W, eps, device=device)
            self.norm2b = WeightOnlyLayerNorm(W, eps, device=device)


class RasodraForCausalLM(nn.Module):
    """``layers`` holds a module for every layer that has tensors of its own (key = its index); ``layer_sequence()`` is
    the list the model runs, in which a layer with ``weights_of`` appears as its owner's module."""

    def __init__(self, config: RasodraConfig, device=None):
        super().__init__()
        self.config = config
        dt = config.torch_dtype
        self.embed_tokens = ParallelEmbedding(config.vocab_size, config.hidden_size, dtype=dt, device=device,
                                              init_method=_init(config.initializer_range))
        self.layers = nn.ModuleDict({str(i): RasodraDecoderLayer(config, L, device=device)
                                     for i, L in enumerate(config.layers) if L.weights_of is None})
        self.norm = WeightOnlyLayerNorm(config.hidden_size, config.rms_norm_eps, device=device)
        self.lm_head = ColumnParallelLinear(config.hidden_size, config.vocab_size, bias=False, gather_output=False,
                                            dtype=dt, device=device, init_method=_init(config.initializer_range))

    def layer_sequence(self) -> List[RasodraDecoderLayer]:
        return [self.layers[str(self.config.owner(i))] for i in range(len(self.config.layers))]


def convert_rasodra_state_dict(sd: Dict[str, torch.Tensor], config: RasodraConfig) -> Dict[str, torch.Tensor]:
    """Checkpoint names (``embed``, ``l<i>.norm1`` ..., ``l<i>.mix.<name>`` / ``<name>.b``, ``l<i>.mlp.up`` / ``down``,
    ``final.norm``, ``head``; linear weights ``[out, in]``) -> this module's state dict."""
    out: Dict[str, torch.Tensor] = {"embed_tokens.weight": sd["embed"], "lm_head.weight": sd["head"],
                                    "norm.weight": sd["final.norm"].float()}
    for i, L in enumerate(config.layers):
        if L.weights_of is not None:
            continue
        src, dst, m = f"l{i}.", f"layers.{i}.", L.mixer
        mix = lambda n: sd[src + "mix." + n]                                          # noqa: E731
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L.mlp is not None else ()):
            out[dst + n + ".weight"] = sd[src + n].float()
        if L.type == "attention":
            out[dst + "mixer.qk_proj.weight"] = torch.cat([mix("q"), mix("k")], dim=0)
            out[dst + "mixer.qk_proj.bias"] = torch.cat([mix("q.b"), mix("k.b")], dim=0)
            out[dst + "mixer.q_norm"] = mix("q.norm").float()
            out[dst + "mixer.k_norm"] = mix("k.norm").float()
        elif L.type == "latent_attention":
            out[dst + "mixer.in_proj.weight"] = torch.cat([mix("q"), mix("dkv"), mix("g")], dim=0)
            out[dst + "mixer.kv_norm"] = mix("dkv.norm").float()
            out[dst + "mixer.uk"] = mix("uk").reshape(m.heads, m.dim, m.kv_rank)
            out[dst + "mixer.uv"] = mix("uv").reshape(m.heads, m.vdim, m.kv_rank)
            out[dst + "mixer.sink"] = mix("sink").float()
        elif L.type == "mlstm":
            out[dst + "mixer.in_proj.weight"] = torch.cat([mix("q"), mix("k"), mix("v"), mix("g")], dim=0)
            out[dst + "mixer.gate_weight"] = torch.cat([mix("i"), mix("f")], dim=0)
            out[dst + "mixer.gate_bias"] = torch.cat([mix("i.b"), mix("f.b")], dim=0).float()
            out[dst + "mixer.out_norm"] = mix("norm").float()
        out[dst + "mixer.o_proj.weight"] = mix("o")
        if L.mlp is not None:
            out[dst + "mlp.up_proj.weight"] = sd[src + "mlp.up"]
            out[dst + "mlp.down_proj.weight"] = sd[src + "mlp.down"]
    return {k: v.contiguous() for k, v in out.items()}


def export_rasodra_state_dict(model: RasodraForCausalLM) -> Dict[str, torch.Tensor]:
    """The inverse of ``convert_rasodra_state_dict``: this module's parameters under the checkpoint names."""
    cfg, sd = model.config, model.state_dict()
    out: Dict[str, torch.Tensor] = {"embed": sd["embed_tokens.weight"], "head": sd["lm_head.weight"],
                                    "final.norm": sd["norm.weight"]}
    for i, L in enumerate(cfg.layers):
        if L.weights_of is not None:
            continue
        src, dst, m = f"layers.{i}.", f"l{i}.", L.mixer
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L.mlp is not None else ()):
            out[dst + n] = sd[src + n + ".weight"]
        if L.type == "attention":
            w, b = sd[src + "mixer.qk_proj.weight"], sd[src + "mixer.qk_proj.bias"]
            nq = m.heads * m.dim
            out[dst + "mix.q"], out[dst + "mix.k"], out[dst + "mix.q.b"], out[dst + "mix.k.b"] = w[:nq], w[nq:], b[:nq], b[nq:]
            out[dst + "mix.q.norm"], out[dst + "mix.k.norm"] = sd[src + "mixer.q_norm"], sd[src + "mixer.k_norm"]
        elif L.type == "latent_attention":
            w = sd[src + "mixer.in_proj.weight"]
            nq, nkv = m.heads * (m.dim + m.rot_dim), m.kv_rank + m.rot_dim
            out[dst + "mix.q"], out[dst + "mix.dkv"], out[dst + "mix.g"] = w[:nq], w[nq:nq + nkv], w[nq + nkv:]
            out[dst + "mix.dkv.norm"] = sd[src + "mixer.kv_norm"]
            out[dst + "mix.uk"] = sd[src + "mixer.uk"].reshape(m.heads * m.dim, m.kv_rank)
            out[dst + "mix.uv"] = sd[src + "mixer.uv"].reshape(m.heads * m.vdim, m.kv_rank)
            out[dst + "mix.sink"] = sd[src + "mixer.sink"]
        elif L.type == "mlstm":
            w, g, gb = sd[src + "mixer.in_proj.weight"], sd[src + "mixer.gate_weight"], sd[src + "mixer.gate_bias"]
            a, c = m.heads * m.dim, m.heads * m.vdim
            out[dst + "mix.q"], out[dst + "mix.k"], out[dst + "mix.v"], out[dst + "mix.g"] = (
                w[:a], w[a:2 * a], w[2 * a:2 * a + c], w[2 * a + c:])
            out[dst + "mix.i"], out[dst + "mix.f"] = g[:m.heads], g[m.heads:]
            out[dst + "mix.i.b"], out[dst + "mix.f.b"] = gb[:m.heads], gb[m.heads:]
            out[dst + "mix.norm"] = sd[src + "mixer.out_norm"]
        out[dst + "mix.o"] = sd[src + "mixer.o_proj.weight"]
        if L.mlp is not None:
            out[dst + "mlp.up"], out[dst + "mlp.down"] = sd[src + "mlp.up_proj.weight"], sd[src + "mlp.down_proj.weight"]
    return {k: v.detach().clone().contiguous() for k, v in out.items()}


def tiny_rasodra(torch_dtype: torch.dtype = torch.float32, **kw) -> RasodraConfig:
    """A small configuration for tests and smoke runs: one layer of every kind (the recurrent one without a
    feed-forward), grouped key/value heads, a chunk of 8 positions, and three layers that run with earlier layers'
    weights."""
    att = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.3, "mask": {"size": 8},
           "rot": {"dims": 8, "base": 10000.0}}
    lat = {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 12, "kv_rank": 24, "scale": 0.25, "rot": {"dims": 4, "base": 5000.0}}
    rec = {"heads": 2, "dim": 12, "vdim": 20, "gate_cap": 9.0}
    ff = {"kind": "dense", "ff": 96}
    d = {"architecture": "Rasodra", "vocab": 144, "width": 40, "norm": {"eps": 1e-6},
         "layers": [{"type": "attention", "mixer": att, "mlp": ff},
                    {"type": "mlstm", "mixer": rec, "mlp": None},
                    {"type": "latent_attention", "mixer": lat, "mlp": ff},
                    {"type": "mlstm", "mixer": rec, "mlp": None, "weights_of": 1},
                    {"type": "attention", "mixer": att, "mlp": ff, "weights_of": 0},
                    {"type": "latent_attention", "mixer": lat, "mlp": ff, "weights_of": 2}]}
    d.update(kw)
    return RasodraConfig.from_dict(d, torch_dtype=torch_dtype)
