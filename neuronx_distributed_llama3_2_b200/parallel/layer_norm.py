"""LayerNorm / RMSNorm whose parameters are tagged for sequence parallelism
(reference ``parallel_layers/layer_norm.py:17-37``).

Under SP every TP rank sees a different sequence slice, so the weight/bias grads
are partial sums that ``allreduce_sequence_parallel_gradients`` (grads.py)
all-reduces over TP; the ``sequence_parallel_enabled`` tag is how they are found.
"""
from __future__ import annotations

import torch

from ..ops import norm as norm_ops


class LayerNorm(torch.nn.LayerNorm):
    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True,
                 sequence_parallel_enabled: bool = False, dtype=torch.float32, device=None):
        super().__init__(normalized_shape, eps=eps, elementwise_affine=elementwise_affine, dtype=dtype, device=device)
        self.sequence_parallel_enabled = sequence_parallel_enabled
        if elementwise_affine:
            setattr(self.weight, "sequence_parallel_enabled", sequence_parallel_enabled)
            setattr(self.bias, "sequence_parallel_enabled", sequence_parallel_enabled)


class RMSNorm(torch.nn.Module):
    """``w * x * rsqrt(mean(x^2) + eps)`` (Llama norm; reference training model
    ``examples/training/llama/modeling_llama_nxd.py:142-149`` does it in fp64 to
    dodge XLA auto-downcast; here: fp32 statistics inside one sm_100a kernel)."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, sequence_parallel_enabled: bool = False,
                 dtype=torch.float32, device=None):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device))
        self.variance_epsilon = eps
        self.sequence_parallel_enabled = sequence_parallel_enabled
        setattr(self.weight, "sequence_parallel_enabled", sequence_parallel_enabled)

    def forward(self, hidden_states: torch.Tensor, residual: torch.Tensor = None) -> torch.Tensor:
        """``rmsnorm(hidden_states)``, or with ``residual``: ``rmsnorm(hidden_states + residual)`` in one kernel."""
        if residual is not None:
            return norm_ops.fused_add_rms_norm(hidden_states, residual, self.weight, self.variance_epsilon)[0]
        return norm_ops.rms_norm(hidden_states, self.weight, self.variance_epsilon)


class ZeroCenteredRMSNorm(torch.nn.Module):
    """``x * rsqrt(mean(x^2) + eps) * (1 + w)``: the weight is stored around zero and kept in fp32; statistics in fp32.
    ``forward`` is the plain norm (a model's final norm); ``add_to(x, y)`` is the post-norm residual update
    ``x += norm(y)`` on an fp32 stream, returning the stream and its rounded copy."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, device=None):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.zeros(hidden_size, dtype=torch.float32, device=device))
        self.variance_epsilon = eps

    def forward(self, hidden_states: torch.Tensor, out_dtype: torch.dtype = None) -> torch.Tensor:
        return norm_ops.rms_norm_offset(hidden_states, self.weight, self.variance_epsilon,
                                        out_dtype or hidden_states.dtype, offset=1.0)

    def add_to(self, stream: torch.Tensor, sublayer_out: torch.Tensor, out_dtype: torch.dtype = None):
        return norm_ops.post_norm_residual_(stream, sublayer_out, self.weight, self.variance_epsilon, out_dtype, offset=1.0)


class WeightOnlyLayerNorm(torch.nn.Module):
    """``(x - mean) / sqrt(var + eps) * w`` (no bias; variance of the deviations), weight and statistics in fp32, for
    models that keep an fp32 residual stream with a norm BEFORE and AFTER every sublayer.  ``forward`` is the plain norm
    of the stream; ``add_to(x, y, next_norm)`` does ``x += self(y)`` in place and, in the same pass, returns
    ``next_norm(x)`` -- the next sublayer's input -- in ``out_dtype``."""

    center = True

    def __init__(self, hidden_size: int, eps: float = 1e-6, device=None):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(hidden_size, dtype=torch.float32, device=device))
        self.variance_epsilon = eps

    def forward(self, stream: torch.Tensor, out_dtype: torch.dtype = None) -> torch.Tensor:
        return norm_ops.norm_chain_(stream, None, None, self.weight, self.variance_epsilon,
                                    out_dtype or stream.dtype, center=self.center)[1]

    def add_to(self, stream: torch.Tensor, sublayer_out: torch.Tensor, next_norm: "WeightOnlyLayerNorm" = None,
               out_dtype: torch.dtype = None):
        return norm_ops.norm_chain_(stream, sublayer_out, self.weight, next_norm.weight if next_norm is not None else None,
                                    self.variance_epsilon, out_dtype, center=self.center)
