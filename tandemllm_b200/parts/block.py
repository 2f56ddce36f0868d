"""How a layer's parts are arranged, and a layer built from a `LayerSpec`.

`prenorm_residual` is the pre-norm block with two residual adds (engine/models/lfm2_moe/ref.py:231-239):

    n = norm_m(h);  h = h + mixer(n);  n = norm_f(h);  h = h + feed_forward(n)

A residual add is fused with the norm that follows it, so a layer receives the previous branch's output as
`pending` (not yet added to the residual stream), and returns its own feed-forward output the same way.

`sandwich_norm_residual` norms every sublayer before and after:

    h = h + norm_mb(mixer(norm_m(h)));  h = h + norm_fb(feed_forward(norm_f(h)))

The norm behind a branch, the residual add and the norm in front of the next sublayer are one kernel where the next
sublayer is in the same layer (`add_normed(..., then=next norm)`); a layer hands nothing pending to the next one, so
that whatever a run order adds to the stream between two layers meets a complete residual.
"""

from __future__ import annotations

from ..config.spec import LayerSpec, PartSpec
from ..kernels import ops
from .base import ARRANGEMENTS, make_part, register_part


@register_part("arrangement", "prenorm_residual")
class PreNormResidual:
    def run(self, layer: "Layer", residual, pending, step, cache, writes_cache: bool = True):
        n = layer.mixer_norm.add_norm(residual, pending)
        d = layer.mixer.forward(n, step, cache, writes_cache=writes_cache)
        ff = layer.feed_forward
        if hasattr(ff, "forward_from"):
            return ff.forward_from(layer.feed_forward_norm, residual, d, step)
        return ff.forward(layer.feed_forward_norm.add_norm(residual, d), step)


@register_part("arrangement", "sandwich_norm_residual")
class SandwichNormResidual:
    def run(self, layer: "Layer", residual, pending, step, cache, writes_cache: bool = True):
        n = layer.mixer_norm.add_norm(residual, pending)
        d = layer.mixer.forward(n, step, cache, writes_cache=writes_cache)
        ff = layer.feed_forward
        if getattr(ff, "absent", False):
            layer.mixer_post_norm.add_normed(residual, d)
            return None
        if hasattr(ff, "router_args"):
            # the norm in front of a routed feed-forward runs its router too: the add first, then that kernel
            layer.mixer_post_norm.add_normed(residual, d)
            out = ff.forward_from(layer.feed_forward_norm, residual, None, step)
        else:
            out = ff.forward(layer.mixer_post_norm.add_normed(residual, d, then=layer.feed_forward_norm), step)
        if isinstance(out, ops.GatedSum):       # a dense part, its gate a row, a routed part: added by the norm's kernel
            layer.feed_forward_post_norm.add_normed(residual, out.dense, gate=out.gate, experts=out.experts)
        else:
            layer.feed_forward_post_norm.add_normed(residual, out)
        return None


class Layer:
    """One layer's parts, built from its spec. The layer knows its parts; no part knows the layer."""

    def __init__(self, spec: LayerSpec, hidden_size: int):
        self.spec = spec
        p = spec.prefix

        def norm(ps: PartSpec):
            name = ps.get("name")
            return make_part("norm", ps, prefix=p + (name + "." if name else ""), size=hidden_size)

        self.mixer_norm = norm(spec.mixer_norm)
        self.feed_forward_norm = norm(spec.feed_forward_norm) if spec.feed_forward_norm else None
        self.mixer_post_norm = norm(spec.mixer_post_norm) if spec.mixer_post_norm else None
        self.feed_forward_post_norm = norm(spec.feed_forward_post_norm) if spec.feed_forward_post_norm else None
        self.mixer = make_part("mixer", spec.mixer, prefix=p, hidden_size=hidden_size)
        self.feed_forward = make_part("feed_forward", spec.feed_forward, prefix=p, hidden_size=hidden_size)
        if spec.arrangement not in ARRANGEMENTS:
            raise ValueError(f"unknown arrangement {spec.arrangement!r}; registered: {', '.join(sorted(ARRANGEMENTS))}")
        self.arrangement = ARRANGEMENTS[spec.arrangement]()

    @property
    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.feed_forward_norm,
                                 self.feed_forward, self.feed_forward_post_norm) if p is not None)

    def weight_specs(self, present=None):
        out = []
        for part in self.parts:
            out += part.weight_specs(present)
        return out

    def bind(self, read, runtime):
        for part in self.parts:
            part.bind(read, runtime)

    def run(self, residual, pending, step, cache, writes_cache: bool = True):
        return self.arrangement.run(self, residual, pending, step, cache, writes_cache)
