"""A matrix memory with exponential gates (xLSTM's mLSTM) as a mixer with a state of its own.

One stacked product gives q | k | v | g | i | f in 32-bit (the two gates' rows are a head each);
the scan kernel walks each request's rows in order from the state its slot holds (memory S
[head_dim, v_head_dim], normaliser n, running maximum m, all float32, cleared when a request
starts) and leaves the state of the request's last row there; then each head's read-out is
divided by its root mean square, times the weight over all heads, times sigmoid(g), and the
output product follows. Prompt portions and single tokens take the same kernel: a step's rows
of one request are a run of the recurrence, however the prompt was cut.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..cache import CacheNeeds, StateSpec
from .base import Part, linear, matrix_named, pad_columns, product_width, stack_rows


class MLSTM(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        w, hd, he = spec.weights, spec.num_heads * spec.head_dim, spec.num_heads * spec.v_head_dim
        return {
            w["q"]: (hd, spec.hidden), w["k"]: (hd, spec.hidden), w["v"]: (he, spec.hidden), w["g"]: (he, spec.hidden),
            w["o"]: (spec.hidden, he), w["norm"]: (he,),
            w["i"]: (spec.num_heads, spec.hidden), w["i_bias"]: (spec.num_heads,),
            w["f"]: (spec.num_heads, spec.hidden), w["f_bias"]: (spec.num_heads,),
        }

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if spec.head_dim > 256:
            raise ValueError(f"mlstm: a key size of {spec.head_dim} is more than the scan kernel's 256")
        if spec.gate_cap <= 0:
            raise ValueError(f"mlstm: gate cap {spec.gate_cap} must be positive")

    def load(self, tensors):
        w = self.spec.weights
        self.w_in = stack_rows(self.ctx, tensors, [w["q"], w["k"], w["v"], w["g"], w["i"], w["f"]], "mlstm")
        self.w_o = pad_columns(self.ctx, matrix_named(self.ctx, tensors, w["o"]))      # the gate kernel writes rows this wide
        dev = self.ctx.device
        self.bias_i = tensors[w["i_bias"]].to(dev).float().contiguous()
        self.bias_f = tensors[w["f_bias"]].to(dev).float().contiguous()
        n = tensors[w["norm"]].to(dev)
        self.norm_weight = n.float() if self.ctx.is_f32 else n.contiguous()

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        return CacheNeeds(state=StateSpec((s.num_heads, K.mlstm_state_floats(s.head_dim, s.v_head_dim))))

    def forward(self, h, batch, cache):
        s = self.spec
        hd, he = s.num_heads * s.head_dim, s.num_heads * s.v_head_dim
        stacked = linear(self.ctx, h, self.w_in, out_dtype=torch.float32, keep_split=True)
        o = K.mlstm_scan(stacked, 0, hd, 2 * hd, 2 * hd + 2 * he, 2 * hd + 2 * he + s.num_heads, self.bias_i, self.bias_f,
                         cache.state(), batch.entry_ranges(), batch.slots, batch.entries, s.num_heads, s.head_dim, s.v_head_dim,
                         s.gate_cap, s.head_dim ** -0.5, s.floor)
        y = K.head_gate(o, stacked, 2 * hd + he, self.norm_weight, True, s.eps, self.ctx.dtype, pad_to=product_width(self.ctx, he))
        return linear(self.ctx, y, self.w_o, keep_split=True)
