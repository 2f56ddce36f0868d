"""The Puripel configuration (`"architecture": "Puripel"`), typed.

A decoder whose layers are listed one by one in config.json; a run of them may be repeated with the same weights. Every
size and every constant that can differ between models of the design is read here and nowhere else; `to_spec()` turns it
into the architecture-neutral `ModelSpec`. A key this reader does not know stops the load with its name.

  config.json       vocab, width, norm: {eps}, layers: [{type, mixer: {...}, mlp: {...} | null}, ...],
                    loop: {start, stop, times} (optional)
  layer             h += norm1b(mixer(norm1 h));  h += norm2b(mlp(norm2 h)): RMS norms with weights `l<i>.norm1`, `.norm1b`,
                    `.norm2`, `.norm2b` (the last two only with an mlp)
  mamba2            mixer: {heads, vdim, state, groups, conv, norm_groups}: the selective state-space mixer; tensors
                    `l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}`
  latent_attention  mixer: {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot: {base, dims}, mask: {size}}: attention
                    over a cached latent with a sliding window and interleaved rotary positions on the rot_dim part;
                    tensors `l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o}`
  mlp               {kind: moe, router: {experts, top, scale, groups: {count, keep}}, expert: {ff, limit},
                    shared: {ff, limit}}: sigmoid-scored experts chosen within the best groups, a correction added for
                    the choice only, and a shared expert behind a sigmoid gate a row; every expert is
                    down(g' sigmoid(1.702 g') (u' + 1)) with g' = min(gate n, limit), u' = clamp(up n, -limit, limit);
                    tensors `l<i>.mlp.{router,correction,e<j>.{gate,up,down},shared.{gate,up,down,sg}}`
  loop              layers start .. stop-1 are run `times` times in a row, each pass with caches and states of its own;
                    before each pass row t of `loop.step` [times, width] is added to the stream
  head              the RMS norm `final.norm`, then the embedding table `embed`
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .spec import LayerSpec, ModelSpec, PartSpec, Site, StreamAdd

ARCHITECTURES = ("Puripel",)
MODEL_TYPES = ("puripel",)

GATE_SLOPE = 1.702          # the design's constants: the slope inside the experts' sigmoid,
WEIGHT_FLOOR = 1e-20        # and what is added to the sum of the chosen scores before the division

TOP_KEYS = {"architecture", "architectures", "model_type", "layers", "loop", "norm", "vocab", "width"}
LAYER_KEYS = {"type", "mixer", "mlp"}
MAMBA_KEYS = {"heads", "vdim", "state", "groups", "conv", "norm_groups"}
LATENT_KEYS = {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot", "mask"}
MLP_KEYS = {"kind", "router", "expert", "shared"}
ROUTER_KEYS = {"experts", "top", "scale", "groups"}


def _only(d: dict, known: set, where: str) -> None:
    unknown = sorted(set(d) - known)
    if unknown:
        raise ValueError(f"Puripel config: {where} has key(s) this engine does not know: {', '.join(unknown)}")


def _need(d: dict, keys, where: str) -> None:
    for k in keys:
        if k not in d:
            raise ValueError(f"Puripel config: {where} lacks the required key {k!r}")


@dataclass
class PuripelLayer:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass
class PuripelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: list[PuripelLayer] = field(default_factory=list)
    loop: dict | None = None
    path: str = ""

    @classmethod
    def from_dict(cls, raw: dict, path: str = "", generation: dict | None = None) -> "PuripelConfig":
        _only(raw, TOP_KEYS, "the top level")
        _need(raw, ("layers", "norm", "vocab", "width"), "the top level")
        _only(raw["norm"], {"eps"}, "norm")
        _need(raw["norm"], ("eps",), "norm")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _only(entry, LAYER_KEYS, where)
            _need(entry, ("type", "mixer"), where)
            kind, m = str(entry["type"]), dict(entry["mixer"])
            if kind == "mamba2":
                _only(m, MAMBA_KEYS, where + ".mixer")
                _need(m, ("heads", "vdim", "state", "groups", "conv", "norm_groups"), where + ".mixer")
            elif kind == "latent_attention":
                _only(m, LATENT_KEYS, where + ".mixer")
                _need(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale"), where + ".mixer")
                if m.get("rot") is not None:
                    _only(m["rot"], {"base", "dims"}, where + ".mixer.rot")
                    _need(m["rot"], ("base", "dims"), where + ".mixer.rot")
                if m.get("mask") is not None:
                    _only(m["mask"], {"size"}, where + ".mixer.mask")
                    _need(m["mask"], ("size",), where + ".mixer.mask")
            else:
                raise ValueError(f"Puripel config: {where}.type {kind!r}: mamba2 and latent_attention are implemented")
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                _only(mlp, MLP_KEYS, where + ".mlp")
                _need(mlp, ("kind", "router", "expert"), where + ".mlp")
                if mlp["kind"] != "moe":
                    raise ValueError(f"Puripel config: {where}.mlp.kind {mlp['kind']!r}: moe is implemented")
                _only(mlp["router"], ROUTER_KEYS, where + ".mlp.router")
                _need(mlp["router"], ("experts", "top"), where + ".mlp.router")
                if mlp["router"].get("groups") is not None:
                    _only(mlp["router"]["groups"], {"count", "keep"}, where + ".mlp.router.groups")
                    _need(mlp["router"]["groups"], ("count", "keep"), where + ".mlp.router.groups")
                for part in ("expert", "shared"):
                    if mlp.get(part) is not None:
                        _only(mlp[part], {"ff", "limit"}, f"{where}.mlp.{part}")
                        _need(mlp[part], ("ff", "limit"), f"{where}.mlp.{part}")
            layers.append(PuripelLayer(kind, m, mlp))
        loop = raw.get("loop")
        if loop is not None:
            loop = dict(loop)
            _only(loop, {"start", "stop", "times"}, "loop")
            _need(loop, ("start", "stop", "times"), "loop")
        cfg = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]), layers=layers,
                  loop=loop, path=path)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ValueError("Puripel config: vocab, width and the number of layers must be positive")
        if self.loop is not None:
            a, b, t = int(self.loop["start"]), int(self.loop["stop"]), int(self.loop["times"])
            if not (0 <= a <= b <= len(self.layers)) or t < 1:
                raise ValueError(f"Puripel config: loop {a}..{b} x {t} over {len(self.layers)} layers")
        for i, layer in enumerate(self.layers):
            if layer.mlp is not None:
                r = layer.mlp["router"]
                if not 0 < int(r["top"]) <= int(r["experts"]):
                    raise ValueError(f"Puripel config: layers[{i}]: top {r['top']} of {r['experts']} experts")
                g = r.get("groups")
                if g and (int(r["experts"]) % int(g["count"]) or not 0 < int(g["keep"]) <= int(g["count"])):
                    raise ValueError(f"Puripel config: layers[{i}]: {r['experts']} experts in {g['count']} groups, "
                                     f"{g['keep']} kept")

    def to_dict(self) -> dict:
        out = {"architecture": ARCHITECTURES[0], "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [{"type": l.type, "mixer": l.mixer, "mlp": l.mlp} for l in self.layers]}
        if self.loop is not None:
            out["loop"] = self.loop
        return out

    def run_order(self) -> tuple[Site, ...]:
        """The layers before the loop once, the looped layers `times` times (each pass's first site also adds the pass's
        row of `loop.step`), then the rest. Every site has a cache or state of its own."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(Site(i) for i in range(n))
        a, b, times = int(self.loop["start"]), int(self.loop["stop"]), int(self.loop["times"])
        sites = [Site(i) for i in range(a)]
        for t in range(times):
            sites += [Site(i, add=StreamAdd("loop.step", t, times) if i == a else None) for i in range(a, b)]
        return tuple(sites + [Site(i) for i in range(b, n)])

    def to_spec(self) -> ModelSpec:
        eps = self.norm_eps

        def norm(name):
            return PartSpec("rmsnorm", {"eps": eps, "tensor": name})

        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "mamba2":
                mixer = PartSpec("selective_state_space", {
                    "heads": int(m["heads"]), "head_dim": int(m["vdim"]), "state": int(m["state"]), "groups": int(m["groups"]),
                    "taps": int(m["conv"]), "norm_groups": int(m["norm_groups"]), "eps": eps, "conv_activation": "silu",
                    "names": {"in": "mix.in", "conv": "mix.conv", "conv_bias": "mix.conv.b", "dt_bias": "mix.dt_bias",
                              "a_log": "mix.A_log", "d": "mix.D", "norm": "mix.norm", "out": "mix.o"}})
            else:
                rot = m.get("rot")
                position = (PartSpec("rope_pairs", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"])})
                            if rot else PartSpec("rope_pairs", {"theta": 1.0, "rotary_dim": 0}))
                mixer = PartSpec("latent_attention", {
                    "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]),
                    "value_dim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]), "q_rank": int(m["q_rank"]),
                    "scale": float(m["scale"]), "window": int(m["mask"]["size"]) if m.get("mask") else None, "eps": eps,
                    "position": position,
                    "names": {"dq": "mix.dq", "dq_norm": "mix.dq.norm", "uq": "mix.uq", "dkv": "mix.dkv",
                              "dkv_norm": "mix.dkv.norm", "uk": "mix.uk", "uv": "mix.uv", "out": "mix.o"}})
            if layer.mlp is None:
                ff = PartSpec("none", {})
            else:
                r, e = layer.mlp["router"], layer.mlp["expert"]
                g = r.get("groups")
                routed = PartSpec("sigmoid_topk_experts", {
                    "num_experts": int(r["experts"]), "top_k": int(r["top"]), "intermediate_size": int(e["ff"]),
                    "expert_bias": True, "normalize": True, "scale": float(r.get("scale", 1.0)), "norm_floor": WEIGHT_FLOOR,
                    "scoring": "sigmoid", "groups": (int(g["count"]), int(g["keep"])) if g else None,
                    "activation": "clamped_swish", "gate_limit": float(e["limit"]), "gate_slope": GATE_SLOPE,
                    "weight_suffix": "", "expert_separator": "",
                    "names": {"router": "mlp.router", "bias": "mlp.correction", "experts": "mlp.e", "gate": "gate", "up": "up",
                              "down": "down"}})
                s = layer.mlp.get("shared")
                if s:
                    shared = PartSpec("swiglu", {
                        "intermediate_size": int(s["ff"]), "activation": "clamped_swish", "gate_limit": float(s["limit"]),
                        "gate_slope": GATE_SLOPE, "weight_suffix": "",
                        "names": {"gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"}})
                    ff = PartSpec("shared_and_routed", {"routed": routed, "shared": shared, "shared_gate": "mlp.shared.sg"})
                else:
                    ff = routed
            has_ff = layer.mlp is not None
            layers.append(LayerSpec(
                prefix=f"l{i}.", mixer=mixer, feed_forward=ff, mixer_norm=norm("norm1"),
                feed_forward_norm=norm("norm2") if has_ff else None, arrangement="sandwich_norm_residual",
                mixer_post_norm=norm("norm1b"), feed_forward_post_norm=norm("norm2b") if has_ff else None))
        return ModelSpec(
            architecture=ARCHITECTURES[0], hidden_size=self.width, vocab_size=self.vocab, layers=tuple(layers),
            schedule=self.run_order(), final_norm=PartSpec("rmsnorm", {"eps": eps, "tensor": "norm"}),
            embedding_name="embed", final_norm_prefix="final.", head_name=None, name_prefixes=())
