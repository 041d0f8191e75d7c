"""Typed configuration of the Gozatar decoder, read from config.json keys.

A Gozatar model is a list of pre-norm layers over ``streams`` copies of the residual stream (hyper-connections; without
the key: one stream and plain residual sums). Every layer names its mixer (``type``: ``parallel`` = a convolved
sliding-window attention and a gated linear attention side by side, reading the same input) with the mixer's sizes,
and its feed-forward (``mlp``: ``{"kind": "dense", "ff": n}`` = the tanh-gelu feed-forward, ``{"kind": "moe", ...}`` =
routed clamped-GLU experts with a shared one, or null for none). Norms are layer norms with a weight and no bias. The
head has a matrix of its own.

config.json keys: ``architecture`` ("Gozatar"), ``vocab``, ``width``, ``streams``, ``norm.eps``,
``layers[i].type | mixer | mlp``; ``mixer.left``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``, ``rot.dims``,
``rot.base``, ``scale``, ``mask.size``; ``mixer.right``: ``heads``, ``dim``, ``vdim``, ``tau`` (and optionally ``rank``:
else the tensors say it); ``mixer.left_scale``, ``mixer.right_scale``; ``mlp.ff`` or ``mlp.expert.ff|limit``,
``mlp.router.experts|top|groups.count|groups.keep``, ``mlp.shared.ff|limit``. Tensor names: ``embed``;
``l<i>.norm1|norm2``; ``l<i>.hc1|hc2.in|out|mix``; ``l<i>.mix.left.q|k|v|o`` with ``.conv``; ``l<i>.mix.right.q|k|v|g|o|
norm|a1|a2|a2.b``; ``l<i>.mlp.up|down`` or ``l<i>.mlp.router|correction|e<j>.gate|up|down|shared.gate|up|down``;
``final.norm``; ``head``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .duzinex import _NUM, _get
from .llama import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, default_schedule

MIXERS = ("parallel",)
GLU_SLOPE = 1.702                 # the design fixes the sigmoid's slope in its experts' activation


def _positive(d: dict, key: str, where: str, optional: bool = False):
    v = _get(d, key, where, optional=optional)
    if v is not None and v <= 0:
        raise ConfigError(f"config.json field {where}{key!r} must be positive, got {v}")
    return v


def _expert(d: dict, where: str) -> dict:
    return dict(ff=_positive(d, "ff", where), limit=float(_get(d, "limit", where, _NUM)))


@dataclass(frozen=True)
class GozatarConfig:
    vocab: int
    width: int
    streams: Optional[int]           # None: one stream, plain residual sums, no hyper-connection tensors
    norm_eps: float
    layers: tuple                    # per layer the validated dict {type, mixer, mlp}
    raw: Optional[dict] = None       # config.json as it was read (written back by ``to_dict``)

    architecture = "Gozatar"

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: dict) -> "GozatarConfig":
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
            lw, rw = where + "mixer.left.", where + "mixer.right."
            l, r = _get(m, "left", where + "mixer.", (dict,)), _get(m, "right", where + "mixer.", (dict,))
            heads = _positive(l, "heads", lw)
            kvh = _positive(l, "kv_heads", lw, optional=True) or heads
            if heads % kvh:
                raise ConfigError(f"{lw}heads {heads} must be a multiple of kv_heads {kvh}")
            dim = _positive(l, "dim", lw)
            left = dict(heads=heads, kv_heads=kvh, dim=dim, vdim=_positive(l, "vdim", lw, optional=True) or dim,
                        conv=_positive(l, "conv", lw, optional=True), scale=float(_get(l, "scale", lw, _NUM)))
            mask = _get(l, "mask", lw, (dict,), optional=True)
            left["window"] = _positive(mask, "size", lw + "mask.") if mask else None
            rot = _get(l, "rot", lw, (dict,), optional=True)
            left["rot_dims"], left["rot_base"] = 0, 10000.0
            if rot:
                dims = _get(rot, "dims", lw + "rot.")
                if dims < 0 or dims % 2 or dims > dim:
                    raise ConfigError(f"{lw}rot.dims {dims} must be even and at most dim {dim}")
                left["rot_dims"], left["rot_base"] = dims, float(_get(rot, "base", lw + "rot.", _NUM))
            right = dict(heads=_positive(r, "heads", rw), dim=_positive(r, "dim", rw), vdim=_positive(r, "vdim", rw),
                         tau=float(_get(r, "tau", rw, _NUM)), rank=_positive(r, "rank", rw, optional=True))
            if not right["tau"] > 0:
                raise ConfigError(f"{rw}tau must be positive")
            mixer = dict(left=left, right=right, left_scale=float(_get(m, "left_scale", where + "mixer.", _NUM)),
                         right_scale=float(_get(m, "right_scale", where + "mixer.", _NUM)))
            # "conv" absent: no convolution and no such tensors; present, even as 1: that many taps
            mlp = layer.get("mlp")
            if mlp is not None:
                mw = where + "mlp."
                mk = _get(mlp, "kind", mw, (str,))
                if mk == "dense":
                    mlp = dict(kind=mk, ff=_positive(mlp, "ff", mw))
                elif mk == "moe":
                    ro = _get(mlp, "router", mw, (dict,))
                    groups = _get(ro, "groups", mw + "router.", (dict,), optional=True)
                    shared = _get(mlp, "shared", mw, (dict,), optional=True)
                    mlp = dict(kind=mk, expert=_expert(_get(mlp, "expert", mw, (dict,)), mw + "expert."),
                               experts=_positive(ro, "experts", mw + "router."), top=_positive(ro, "top", mw + "router."),
                               groups=_positive(groups, "count", mw + "router.groups.") if groups else 1,
                               keep=_positive(groups, "keep", mw + "router.groups.") if groups else 1,
                               shared=_expert(shared, mw + "shared.") if shared else None)
                    if mlp["experts"] % mlp["groups"] or mlp["keep"] > mlp["groups"]:
                        raise ConfigError(f"{mw}router: {mlp['experts']} experts, {mlp['groups']} groups, {mlp['keep']} kept "
                                          "do not fit together")
                    allowed = mlp["experts"] if mlp["groups"] == 1 else mlp["keep"] * (mlp["experts"] // mlp["groups"])
                    if mlp["top"] > allowed:
                        raise ConfigError(f"{mw}router.top {mlp['top']} is more than the {allowed} experts that can be chosen")
                else:
                    raise ConfigError(f"config.json field {mw}'kind' is {mk!r}; known: 'dense', 'moe'")
            checked.append(dict(type=kind, mixer=mixer, mlp=mlp))
        norm = d.get("norm") or {}
        cfg = cls(vocab=_positive(d, "vocab", ""), width=_positive(d, "width", ""),
                  streams=_positive(d, "streams", "", optional=True),
                  norm_eps=float(_get(norm, "eps", "norm.", _NUM)), layers=tuple(checked), raw=dict(d))
        return cfg

    def to_dict(self) -> dict:
        if self.raw is not None:
            return dict(self.raw)
        layers = []
        for l in self.layers:
            left = {k: v for k, v in l["mixer"]["left"].items() if v is not None}
            w, rd, rb = left.pop("window", None), left.pop("rot_dims"), left.pop("rot_base")
            if w:
                left["mask"] = dict(size=w)
            if rd:
                left["rot"] = dict(dims=rd, base=rb)
            right = {k: v for k, v in l["mixer"]["right"].items() if v is not None}
            mlp = l["mlp"]
            if mlp is not None and mlp["kind"] == "moe":
                mlp = dict(kind="moe", expert=dict(mlp["expert"]), shared=dict(mlp["shared"]) if mlp["shared"] else None,
                           router=dict(experts=mlp["experts"], top=mlp["top"],
                                       groups=dict(count=mlp["groups"], keep=mlp["keep"])))
            layers.append(dict(type=l["type"], mlp=mlp,
                               mixer=dict(left=left, right=right, left_scale=l["mixer"]["left_scale"],
                                          right_scale=l["mixer"]["right_scale"])))
        out = dict(architecture=self.architecture, vocab=self.vocab, width=self.width, norm=dict(eps=self.norm_eps),
                   layers=layers)
        if self.streams:
            out["streams"] = self.streams
        return out

    def stop_token_ids(self) -> list:
        return []

    # ------------------------------------------------------------------ model
    def to_spec(self) -> ModelSpec:
        W, S, eps = self.width, self.streams, self.norm_eps

        def norm(prefix, streams=1):
            return PartSpec("layernorm", dict(size=W, eps=eps, weight_name="", streams=streams), prefix=prefix)

        layers = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.", l["mixer"]
            a, g = m["left"], m["right"]
            rope = None
            if a["rot_dims"] > 0:
                rope = PartSpec("rotary", dict(theta=a["rot_base"], rotary_dim=a["rot_dims"]))
            left = PartSpec("conv_attention", dict(
                hidden_size=W, num_heads=a["heads"], num_kv_heads=a["kv_heads"], head_dim=a["dim"], v_head_dim=a["vdim"],
                conv_taps=a["conv"], scale=a["scale"], qk_norm_eps=eps, out_scale=m["left_scale"], position=rope,
                window=a["window"]), prefix=p + "mix.left.")
            right = PartSpec("gla", dict(hidden_size=W, num_heads=g["heads"], dim=g["dim"], vdim=g["vdim"], tau=g["tau"],
                                         eps=eps, rank=g["rank"], out_scale=m["right_scale"]), prefix=p + "mix.right.")
            mixer = PartSpec("parallel", dict(left=left, right=right), prefix=p + "mix.")
            ffn, f = None, l["mlp"]
            if f is not None and f["kind"] == "dense":
                ffn = PartSpec("gelu_mlp", dict(hidden_size=W, intermediate_size=f["ff"]), prefix=p + "mlp.")
            elif f is not None:
                shared = None
                if f["shared"]:
                    shared = PartSpec("clamped_glu", dict(hidden_size=W, intermediate_size=f["shared"]["ff"],
                                                          limit=f["shared"]["limit"], slope=GLU_SLOPE), prefix=p + "mlp.shared.")
                ffn = PartSpec("routed_experts", dict(
                    hidden_size=W, intermediate_size=f["expert"]["ff"], experts=f["experts"], top=f["top"],
                    limit=f["expert"]["limit"], slope=GLU_SLOPE, groups=f["groups"], keep_groups=f["keep"], shared=shared),
                    prefix=p + "mlp.")
            norms = {"mixer": norm(p + "norm1"), "ffn": norm(p + "norm2")}
            if S:
                layers.append(LayerSpec(block="hyper", mixer=mixer, ffn=ffn, norms=norms,
                                        params=dict(hidden_size=W, streams=S, prefix=p)))
            else:
                layers.append(LayerSpec(block="prenorm", mixer=mixer, ffn=ffn, norms=norms))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=W,
            embedding=PartSpec("embedding", dict(vocab_size=self.vocab, hidden_size=W, weight_name="embed")),
            layers=tuple(layers), schedule=default_schedule(len(layers)), final_norm=norm("final.norm", S or 1),
            head=PartSpec("lm_head", dict(vocab_size=self.vocab, hidden_size=W, weight_name="head")),
            max_position=0, streams=S or 1)
        spec.validate()
        return spec


register_architecture(GozatarConfig.architecture, GozatarConfig)
