"""The gated delta rule as a mixer with a state of its own.

One stacked product gives q | k | v | g | b | a in 32-bit (b and a: a column a head). The scan's
kernels convolve q, k and v over the last rows per channel (the rows before this step come from the
request's slot), apply silu, make q and k unit vectors, compute the decay and the step size, and
walk each request's rows in order from the memory its slot holds, leaving the memory of the
request's last row and the convolutions' newest inputs there. Then each head's read-out is divided
by its root mean square, times a weight shared by the heads, times silu(g), and the output product
follows. Prompt portions and single tokens take the same kernels: a step's rows of one request are
a run of the recurrence, however the prompt was cut.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..cache import CacheNeeds, StateSpec
from .base import Part, linear, matrix_named, pad_columns, product_width, stack_rows


class Delta(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        w = spec.weights
        kd, he = spec.num_kv_heads * spec.head_dim, spec.num_heads * spec.v_head_dim
        return {
            w["q"]: (kd, spec.hidden), w["k"]: (kd, spec.hidden), w["v"]: (he, spec.hidden), w["g"]: (he, spec.hidden),
            w["q_conv"]: (kd, spec.conv), w["k_conv"]: (kd, spec.conv), w["v_conv"]: (he, spec.conv),
            w["b"]: (spec.num_heads, spec.hidden), w["a"]: (spec.num_heads, spec.hidden),
            w["A_log"]: (spec.num_heads,), w["dt_bias"]: (spec.num_heads,), w["norm"]: (spec.v_head_dim,),
            w["o"]: (spec.hidden, he),
        }

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"delta: {spec.num_heads} heads over {spec.num_kv_heads} key heads")
        if spec.head_dim > 256:
            raise ValueError(f"delta: a key size of {spec.head_dim} is more than the scan kernel's 256")
        if not 1 <= spec.conv <= 8:
            raise ValueError(f"delta: a convolution over {spec.conv} rows (1 to 8)")

    def load(self, tensors):
        s, w = self.spec, self.spec.weights
        self.w_in = stack_rows(self.ctx, tensors, [w["q"], w["k"], w["v"], w["g"], w["b"], w["a"]], "delta")
        self.w_o = pad_columns(self.ctx, matrix_named(self.ctx, tensors, w["o"]))      # the gate kernel writes rows this wide
        dev = self.ctx.device
        f32 = lambda n: tensors[n].to(dev).float().contiguous()
        self.conv = torch.cat([f32(w["q_conv"]), f32(w["k_conv"]), f32(w["v_conv"])], dim=0).contiguous()
        self.a_log, self.dt_bias = f32(w["A_log"]), f32(w["dt_bias"])
        n = tensors[w["norm"]].to(dev)
        n = n.float() if self.ctx.is_f32 else n
        self.norm_weight = n.repeat(s.num_heads).contiguous()                           # one weight for all heads

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        return CacheNeeds(state=StateSpec((K.delta_state_floats(s.num_heads, s.num_kv_heads, s.head_dim, s.v_head_dim, s.conv),)))

    def forward(self, h, batch, cache):
        s = self.spec
        kd, he = s.num_kv_heads * s.head_dim, s.num_heads * s.v_head_dim
        stacked = linear(self.ctx, h, self.w_in, out_dtype=torch.float32, keep_split=True)
        o = K.delta_scan(stacked, 0, kd, 2 * kd, 2 * kd + 2 * he, 2 * kd + 2 * he + s.num_heads, self.conv, self.a_log, self.dt_bias,
                         cache.state(), batch.row_entry, batch.entry_ranges(), batch.slots, batch.entries, s.num_heads, s.num_kv_heads,
                         s.head_dim, s.v_head_dim, s.conv, s.head_dim ** -0.5, s.unit_eps)
        y = K.head_gate(o, stacked, 2 * kd + he, self.norm_weight, True, s.eps, self.ctx.dtype, pad_to=product_width(self.ctx, he),
                        gate_act="silu")
        return linear(self.ctx, y, self.w_o, keep_split=True)
