"""The Sifupel configuration (`"architecture": "Sifupel"`), typed.

A decoder whose layers are listed one by one in config.json: each entry names its mixer's type, the mixer's sizes and
its feed-forward (or none). Every size and every constant that can differ between models of the design is read here and
nowhere else; `to_spec()` turns it into the architecture-neutral `ModelSpec`. A key this reader does not know stops
the load with its name.

  config.json   vocab, width, norm: {eps}, layers: [{type, mixer: {...}, mlp: {kind, ff} | null}, ...]
  attention     mixer: {heads, kv_heads, dim, vdim, scale, mask: {size}}: sliding-window attention without a position
                encoding; q and k at unit root mean square per head; the values are the keys as projected; the heads'
                softmax weights mixed by `mix.talk`; a sigmoid gate a head (`mix.g`); tensors `l<i>.mix.{q,k,talk,g,o}`
  dense         mlp: {kind: dense, ff}: down(xielu(up n)), tensors `l<i>.mlp.{up,down,act}`
  norms         Dynamic Tanh: `l<i>.norm1`, `l<i>.norm2`, `final.norm`, each with `.b` and `.alpha`
  head          the embedding table `embed`
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .spec import LayerSpec, ModelSpec, PartSpec, plain_schedule

ARCHITECTURES = ("Sifupel",)
MODEL_TYPES = ("sifupel",)

TOP_KEYS = {"architecture", "architectures", "model_type", "layers", "norm", "vocab", "width"}
LAYER_KEYS = {"type", "mixer", "mlp"}
ATTENTION_KEYS = {"heads", "kv_heads", "dim", "vdim", "scale", "mask"}
MLP_KEYS = {"kind", "ff"}


def _only(d: dict, known: set, where: str) -> None:
    unknown = sorted(set(d) - known)
    if unknown:
        raise ValueError(f"Sifupel config: {where} has key(s) this engine does not know: {', '.join(unknown)}")


def _need(d: dict, keys, where: str) -> None:
    for k in keys:
        if k not in d:
            raise ValueError(f"Sifupel config: {where} lacks the required key {k!r}")


@dataclass
class SifupelLayer:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass
class SifupelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: list[SifupelLayer] = field(default_factory=list)
    path: str = ""

    @classmethod
    def from_dict(cls, raw: dict, path: str = "", generation: dict | None = None) -> "SifupelConfig":
        _only(raw, TOP_KEYS, "the top level")
        _need(raw, ("layers", "norm", "vocab", "width"), "the top level")
        _only(raw["norm"], {"eps"}, "norm")
        _need(raw["norm"], ("eps",), "norm")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _only(entry, LAYER_KEYS, where)
            _need(entry, ("type", "mixer"), where)
            kind = str(entry["type"])
            m = dict(entry["mixer"])
            if kind == "attention":
                _only(m, ATTENTION_KEYS, where + ".mixer")
                _need(m, ("heads", "kv_heads", "dim", "vdim", "scale", "mask"), where + ".mixer")
                _only(m["mask"], {"size"}, where + ".mixer.mask")
                _need(m["mask"], ("size",), where + ".mixer.mask")
            else:
                raise ValueError(f"Sifupel config: {where}.type {kind!r}: attention is implemented")
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                _only(mlp, MLP_KEYS, where + ".mlp")
                _need(mlp, ("kind", "ff"), where + ".mlp")
                if mlp["kind"] != "dense":
                    raise ValueError(f"Sifupel config: {where}.mlp.kind {mlp['kind']!r}: dense is implemented")
            layers.append(SifupelLayer(kind, m, mlp))
        cfg = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]), layers=layers,
                  path=path)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ValueError("Sifupel config: vocab, width and the number of layers must be positive")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            H, G, D, VD = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            if H <= 0 or G <= 0 or H % G:
                raise ValueError(f"Sifupel config: layers[{i}]: {H} heads are not a multiple of {G} kv_heads")
            if VD != D:
                raise ValueError(f"Sifupel config: layers[{i}]: the values are the keys, so vdim ({VD}) must equal dim ({D})")
            if D <= 0 or int(m["mask"]["size"]) <= 0:
                raise ValueError(f"Sifupel config: layers[{i}]: dim and mask.size must be positive")
            if layer.mlp is not None and int(layer.mlp["ff"]) <= 0:
                raise ValueError(f"Sifupel config: layers[{i}]: mlp.ff must be positive")

    def to_dict(self) -> dict:
        return {"architecture": ARCHITECTURES[0], "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "layers": [{"type": l.type, "mixer": l.mixer, "mlp": l.mlp} for l in self.layers]}

    def to_spec(self) -> ModelSpec:
        eps = self.norm_eps
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            mixer = PartSpec("attention", {
                "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]), "head_dim": int(m["dim"]),
                "qk_norm": PartSpec("unit_rms", {"eps": eps}), "position": PartSpec("none", {}),
                "scale": float(m["scale"]), "window": int(m["mask"]["size"]), "values": "keys",
                "head_mix": "mix.talk", "gate": "mix.g", "weight_suffix": "",
                "names": {"q": "mix.q", "k": "mix.k", "out": "mix.o"},
            })
            if layer.mlp is None:
                ff = PartSpec("none", {})
            else:
                ff = PartSpec("dense_act", {"intermediate_size": int(layer.mlp["ff"]), "activation": "xielu",
                                            "names": {"up": "mlp.up", "down": "mlp.down", "act_params": "mlp.act"}})
            layers.append(LayerSpec(
                prefix=f"l{i}.", mixer=mixer, feed_forward=ff,
                mixer_norm=PartSpec("dyt", {"eps": eps, "name": "norm1"}),
                feed_forward_norm=PartSpec("dyt", {"eps": eps, "name": "norm2", "optional": layer.mlp is None})))
        return ModelSpec(
            architecture=ARCHITECTURES[0], hidden_size=self.width, vocab_size=self.vocab, layers=tuple(layers),
            schedule=plain_schedule(len(layers)), final_norm=PartSpec("dyt", {"eps": eps}),
            embedding_name="embed", final_norm_prefix="final.norm.", head_name=None, name_prefixes=())
