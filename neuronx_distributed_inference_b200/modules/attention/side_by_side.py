"""Two sequence mixers side by side on one input: one stacked input projection, two results, and how the block is to combine them.

``left`` and ``right`` are mixers built with ``own_in_proj=False`` (``in_width`` projection rows each, ``forward_projected(p, meta,
kv_mgr, cache_index)``): an attention layer beside a recurrent one, for instance.  ``in_proj`` stacks their projection rows
``[left | right]`` so that both read the normalised stream through ONE GEMM.  The results are not summed here: the module returns a
:class:`MixerPair` that says how they combine,

    y = left_scale * f(left) + right_scale * f(right),      f(v) = rms_unit(v) * out_weight  when ``out_norm``, else v

and the block's stream kernel (``ops.stream_sandwich_norm``) forms ``y`` in fp32 together with the norms and the sum that follow, so
nothing between the two output projections and the residual stream is rounded.  ``out_norm=True`` gives each side a learned weight over
the model width (``left_out_weight`` / ``right_out_weight``); the scales are plain constants.
"""
from __future__ import annotations

from typing import NamedTuple, Optional

import torch
import torch.nn as nn

from ...parallel.layers import ColumnParallelLinear


class MixerPair(NamedTuple):
    a: torch.Tensor
    b: Optional[torch.Tensor] = None
    a_weight: Optional[torch.Tensor] = None
    b_weight: Optional[torch.Tensor] = None
    a_scale: float = 1.0
    b_scale: float = 1.0


class SideBySideMixer(nn.Module):
    def __init__(self, hidden_size: int, left: nn.Module, right: nn.Module, *, left_scale: float = 1.0, right_scale: float = 1.0,
                 out_norm: bool = False, dtype=torch.bfloat16, device=None, tp_group=None):
        super().__init__()
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self.in_proj = ColumnParallelLinear(hidden_size, left.in_width + right.in_width, bias=False, gather_output=False, dtype=dtype,
                                            device=device, tensor_model_parallel_group=tp_group)
        w = lambda: nn.Parameter(torch.ones(hidden_size, dtype=torch.float32, device=device), requires_grad=False)      # noqa: E731
        self.left_out_weight = w() if out_norm else None
        self.right_out_weight = w() if out_norm else None

    def state_specs(self, cache_index=None):
        specs = dict(self.left.state_specs(cache_index))
        specs.update(self.right.state_specs(cache_index))
        return specs

    def kv_shape(self):
        """The pair's cache is that of whichever side keeps one (attention beside a recurrent mixer)."""
        for m in (self.left, self.right):
            shape = getattr(m, "kv_shape", lambda: None)()
            if shape is not None:
                return shape
        return None

    def forward(self, x, meta, kv_mgr, cache_index=None) -> MixerPair:
        p = self.in_proj(x)
        nl = self.left.in_width
        a = self.left.forward_projected(p[..., :nl], meta, kv_mgr, cache_index)
        b = self.right.forward_projected(p[..., nl:], meta, kv_mgr, cache_index)
        return MixerPair(a, b, self.left_out_weight, self.right_out_weight, self.left_scale, self.right_scale)
