"""The selective state-space mixer (the Mamba-2 recurrence) with a fixed-size per-request state.

  [z | x | B | C | dt] = in_proj(n)         z, x: heads * cols entries; B, C: groups * state entries each; dt: one a head
  x, B, C <- act(causal depthwise conv over the last `taps` tokens + bias)
  dt = softplus(dt + dt_bias);  per head h, with the B and C of its group:
      S <- exp(-exp(A_log[h]) dt) S + dt B x^T          S: state x cols, zero for a new sequence
      y = S^T C + D[h] x
  out = out_proj( norm_weight * v / rms(v) in `norm_groups` equal parts of a row ),  v = y * silu(z)

A request's slot holds, in 32-bit, the last taps - 1 inputs of the convolution and then the heads' recurrent states. The
in-projection's result is kept in 32-bit in both precisions: the step sizes, decays, B, C and x enter the recurrence
unrounded. Rows of several requests run side by side, a request's rows one after the other (csrc/ssm.cu); a portion of
any length starts from the slot and leaves it as the next portion needs it.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part, SlotNeed, register_part
from .linear import linear


@register_part("mixer", "selective_state_space")
class SelectiveStateSpaceMixer(Part):
    graph_safe = True

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.heads, self.cols, self.n_state = int(spec["heads"]), int(spec["head_dim"]), int(spec["state"])
        self.groups, self.taps, self.norm_groups = int(spec["groups"]), int(spec["taps"]), int(spec.get("norm_groups", 1))
        self.eps = float(spec["eps"])
        self.conv_act = str(spec.get("conv_activation", "silu"))
        self.inner = self.heads * self.cols
        self.channels = self.inner + 2 * self.groups * self.n_state          # what the convolution runs over: x, B, C
        self.proj = 2 * self.inner + 2 * self.groups * self.n_state + self.heads
        if self.heads <= 0 or self.groups <= 0 or self.heads % self.groups:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.groups} groups")
        if self.norm_groups <= 0 or self.inner % self.norm_groups:
            raise ValueError(f"rows of {self.inner} do not fall into {self.norm_groups} equal parts")
        if not 1 <= self.taps <= 64:
            raise ValueError(f"a convolution of {self.taps} taps: 1 to 64 are implemented")
        if not 1 <= self.n_state <= 256:
            raise ValueError(f"a state of {self.n_state} rows a head: 1 to 256 are implemented")
        self.n = {k: prefix + v for k, v in spec["names"].items()}
        self.conv_floats = (self.taps - 1) * self.channels

    def weight_specs(self, present=None):
        n, H = self.n, self.heads
        return [TensorSpec(n["in"], (self.proj, self.hidden_size)),
                TensorSpec(n["conv"], (self.channels, self.taps), "vector", "bias"),
                TensorSpec(n["conv_bias"], (self.channels,), "vector", "bias"),
                TensorSpec(n["dt_bias"], (H,), "vector", "bias"), TensorSpec(n["a_log"], (H,), "vector", "bias"),
                TensorSpec(n["d"], (H,), "vector", "ones"), TensorSpec(n["norm"], (self.inner,), "vector", "ones"),
                TensorSpec(n["out"], (self.hidden_size, self.inner))]

    def bind(self, read, runtime):
        self.runtime = runtime
        n = self.n
        self.w_in = runtime.matrix(read(n["in"]))
        self.w_out = runtime.matrix(read(n["out"]))
        self.w_conv = runtime.vector(read(n["conv"])).reshape(self.channels, self.taps).contiguous()
        self.b_conv = runtime.vector(read(n["conv_bias"]))
        self.dt_bias = runtime.vector(read(n["dt_bias"]))
        self.a_log = runtime.vector(read(n["a_log"]))
        self.d_skip = runtime.vector(read(n["d"]))
        self.w_norm = runtime.vector(read(n["norm"]))

    def cache_need(self):
        return SlotNeed((self.conv_floats + self.heads * self.cols * self.n_state,), torch.float32)

    def forward(self, x, step, cache, writes_cache: bool = True):
        R, dev = x.shape[0], x.device
        inner = self.inner
        proj = linear(self.runtime, x, self.w_in, out_dtype=torch.float32)
        xbc_in = proj[:, inner:]
        xbc = torch.empty(R, self.channels, dtype=torch.float32, device=dev)
        ops.causal_conv_act(xbc_in, self.channels, self.w_conv, self.b_conv, cache.state, step.state_slot, step.req_of_row,
                            step.row_start, xbc, self.conv_act)
        if writes_cache:
            ops.conv_state(xbc_in, self.channels, self.taps, cache.state, step.state_slot, step.row_start, step.n_requests)
        y = torch.empty(R, inner, dtype=torch.float32, device=dev)
        ops.ssm_scan(xbc, proj[:, inner + self.channels:], self.dt_bias, self.a_log, self.d_skip, cache.state, self.conv_floats,
                     step.state_slot, step.row_start, step.n_requests, y, self.heads, self.cols, self.n_state, self.groups,
                     write_state=writes_cache, max_rows_per_request=step.max_rows_per_request, runtime=self.runtime)
        v = torch.empty(R, inner, dtype=x.dtype, device=dev)
        ops.gated_group_norm(y, proj, self.w_norm, self.eps, self.norm_groups, v)
        return linear(self.runtime, v, self.w_out, out_dtype=torch.float32, defer=True)
