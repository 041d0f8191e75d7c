"""Typed configuration of the Duzinex decoder, read from config.json keys.

A Duzinex model is a list of pre-norm layers with a token shift in front of each mixer; every layer names its
mixer (``type``: ``attention`` = differential attention with a sliding window that keeps the first tokens,
``retention``, ``mingru``) with the mixer's sizes, and its feed-forward (``mlp``: ``{"kind": "dense", "ff": n}``
= the PolyNorm feed-forward, or null for none). Norms are dynamic tanh. ``loop`` = {start, stop, times} runs the
layers start … stop−1 ``times`` times in a row with the same weights; each pass has caches and states of its own
and, from the second pass on, takes the embedding's output in again in front of its first layer. The head is the
embedding table itself (without ``embedding.scale``).

config.json keys: ``architecture`` ("Duzinex"), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``,
``layers[i].type | mixer | mlp``, ``loop``. Tensor names: ``embed``; ``l<i>.norm1|norm2`` with ``.b`` and
``.alpha``; ``l<i>.shift``; ``l<i>.mix.*``; ``l<i>.mlp.up|down|act``; ``final.norm``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .llama import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXERS = ("attention", "retention", "mingru")


def _get(d: dict, key: str, where: str, kinds=(int,), optional: bool = False):
    v = d.get(key) if isinstance(d, dict) else None
    if v is None:
        if optional:
            return None
        raise ConfigError(f"config.json is missing required field {where}{key!r}")
    if isinstance(v, bool) or not isinstance(v, kinds):
        raise ConfigError(f"config.json field {where}{key!r} has the wrong type: {v!r}")
    return v


_NUM = (int, float)


@dataclass(frozen=True)
class DuzinexConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple                    # per layer the validated dict {type, mixer, mlp}
    loop_start: int
    loop_stop: int
    loop_times: int
    raw: Optional[dict] = None       # config.json as it was read (written back by ``to_dict``)

    architecture = "Duzinex"

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: dict) -> "DuzinexConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json field 'layers' must be a non-empty list")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            kind = _get(layer, "type", where, (str,))
            if kind not in MIXERS:
                raise ConfigError(f"config.json field {where}'type' is {kind!r}; known mixers: {MIXERS}")
            m = _get(layer, "mixer", where, (dict,))
            mw = where + "mixer."
            if kind == "attention":
                heads, kvh = _get(m, "heads", mw), _get(m, "kv_heads", mw, optional=True) or _get(m, "heads", mw)
                if heads <= 0 or kvh <= 0 or heads % kvh:
                    raise ConfigError(f"{mw}heads {heads} must be a positive multiple of kv_heads {kvh}")
                dim = _get(m, "dim", mw)
                if dim <= 0:
                    raise ConfigError(f"{mw}dim {dim} must be positive")
                mixer = dict(heads=heads, kv_heads=kvh, dim=dim, vdim=_get(m, "vdim", mw),
                             diff=float(_get(m, "diff", mw, _NUM)), scale=float(_get(m, "scale", mw, _NUM)),
                             softcap=_get(m, "softcap", mw, _NUM, optional=True))
                mask = _get(m, "mask", mw, (dict,), optional=True)
                mixer["window"] = _get(mask, "size", mw + "mask.") if mask else None
                mixer["keep_first"] = (_get(mask, "keep_first", mw + "mask.", optional=True) or 0) if mask else 0
                if mixer["window"] is not None and mixer["window"] <= 0:
                    raise ConfigError(f"{mw}mask.size must be positive")
                rot = _get(m, "rot", mw, (dict,), optional=True)
                if rot:
                    dims = _get(rot, "dims", mw + "rot.")
                    if dims < 0 or dims % 2 or dims > dim:
                        raise ConfigError(f"{mw}rot.dims {dims} must be even and at most dim {dim}")
                    mixer["rot_dims"], mixer["rot_base"] = dims, float(_get(rot, "base", mw + "rot.", _NUM))
                else:
                    mixer["rot_dims"], mixer["rot_base"] = 0, 10000.0
            elif kind == "retention":
                heads = _get(m, "heads", mw)
                decay = _get(m, "decay", mw, (list,))
                if len(decay) != heads or any(isinstance(g, bool) or not isinstance(g, _NUM) for g in decay):
                    raise ConfigError(f"{mw}decay must list one number per head ({heads})")
                mixer = dict(heads=heads, dim=_get(m, "dim", mw), vdim=_get(m, "vdim", mw), decay=[float(g) for g in decay])
            else:
                mixer = dict(width=_get(m, "width", mw))
            for k, v in mixer.items():
                if k in ("heads", "dim", "vdim", "width") and v <= 0:
                    raise ConfigError(f"{mw}{k} must be positive, got {v}")
            mlp = layer.get("mlp")
            if mlp is not None:
                mk = _get(mlp, "kind", where + "mlp.", (str,))
                if mk != "dense":
                    raise ConfigError(f"config.json field {where}mlp.'kind' is {mk!r}; known: 'dense'")
                mlp = dict(kind=mk, ff=_get(mlp, "ff", where + "mlp."))
                if mlp["ff"] <= 0:
                    raise ConfigError(f"{where}mlp.ff must be positive")
            checked.append(dict(type=kind, mixer=mixer, mlp=mlp))
        loop = d.get("loop") or {}
        start = _get(loop, "start", "loop.") if loop else 0
        stop = _get(loop, "stop", "loop.") if loop else 0
        times = _get(loop, "times", "loop.") if loop else 1
        if not (0 <= start <= stop <= len(checked)) or times < 1:
            raise ConfigError(f"loop {{start {start}, stop {stop}, times {times}}} does not fit {len(checked)} layers")
        emb = d.get("embedding") or {}
        norm = d.get("norm") or {}
        cfg = cls(vocab=_get(d, "vocab", ""), width=_get(d, "width", ""),
                  embedding_scale=float(_get(emb, "scale", "embedding.", _NUM, optional=True) or 1.0),
                  norm_eps=float(_get(norm, "eps", "norm.", _NUM)), layers=tuple(checked),
                  loop_start=start, loop_stop=stop, loop_times=times, raw=dict(d))
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("vocab and width must be positive")
        return cfg

    def to_dict(self) -> dict:
        if self.raw is not None:
            return dict(self.raw)
        layers = []
        for l in self.layers:
            m = dict(l["mixer"])
            if l["type"] == "attention":
                m["mask"] = dict(size=m.pop("window"), keep_first=m.pop("keep_first")) if m.get("window") else None
                m.pop("window", None), m.pop("keep_first", None)
                m["rot"] = dict(dims=m.pop("rot_dims"), base=m.pop("rot_base"))
            layers.append(dict(type=l["type"], mixer=m, mlp=l["mlp"]))
        return dict(architecture=self.architecture, vocab=self.vocab, width=self.width,
                    embedding=dict(scale=self.embedding_scale), norm=dict(eps=self.norm_eps), layers=layers,
                    loop=dict(start=self.loop_start, stop=self.loop_stop, times=self.loop_times))

    def stop_token_ids(self) -> list:
        return []

    # ------------------------------------------------------------------ model
    def layer_runs(self) -> list:
        """[(layer, takes the embedding in again)] in the order the layers run within a step."""
        runs = [(i, False) for i in range(self.loop_start)]
        for p in range(self.loop_times):
            runs += [(i, p > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return runs + [(i, False) for i in range(self.loop_stop, len(self.layers))]

    def to_spec(self) -> ModelSpec:
        W = self.width

        def norm(prefix):
            return PartSpec("dyt", dict(size=W, weight_name="", bias_name=".b", alpha_name=".alpha"), prefix=prefix)

        layers = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.", l["mixer"]
            if l["type"] == "attention":
                rope = None
                if m["rot_dims"] > 0:
                    rope = PartSpec("rotary", dict(theta=m["rot_base"], rotary_dim=m["rot_dims"], pairing="interleaved"))
                mixer = PartSpec("diff_attention", dict(
                    hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"],
                    diff=m["diff"], scale=m["scale"], eps=self.norm_eps, softcap=m["softcap"], window=m["window"],
                    keep_first=m["keep_first"], position=rope, bias=True), prefix=p + "mix.")
            elif l["type"] == "retention":
                mixer = PartSpec("retention", dict(hidden_size=W, num_heads=m["heads"], dim=m["dim"], vdim=m["vdim"],
                                                   decay=tuple(m["decay"]), eps=self.norm_eps), prefix=p + "mix.")
            else:
                mixer = PartSpec("mingru", dict(hidden_size=W, width=m["width"]), prefix=p + "mix.")
            ffn = None
            if l["mlp"] is not None:
                ffn = PartSpec("polynorm", dict(hidden_size=W, intermediate_size=l["mlp"]["ff"], eps=self.norm_eps),
                               prefix=p + "mlp.")
            layers.append(LayerSpec(block="prenorm_shift", mixer=mixer, ffn=ffn,
                                    norms={"mixer": norm(p + "norm1"), "ffn": norm(p + "norm2")},
                                    params=dict(hidden_size=W, shift_name=p + "shift")))
        schedule = tuple(ScheduleEntry(layer, run, True, again) for run, (layer, again) in enumerate(self.layer_runs()))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=W,
            embedding=PartSpec("embedding", dict(vocab_size=self.vocab, hidden_size=W, weight_name="embed",
                                                 scale=self.embedding_scale)),
            layers=tuple(layers), schedule=schedule, final_norm=norm("final.norm"),
            head=PartSpec("lm_head", dict(vocab_size=self.vocab, hidden_size=W, tied_to="embed")),
            max_position=0)
        spec.validate()
        return spec


register_architecture(DuzinexConfig.architecture, DuzinexConfig)
