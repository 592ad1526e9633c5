"""Mapalorn: a decoder of parallel layers, listed one by one in ``config.json``, a run of which may loop.

A layer is ``h = LN(x); x += mixer(h) + ff(h)``: one layer norm (weight and bias), and both sub-layers read its output
(``kairyu_b200/parts/block.py``: ``parallel``).  The mixer is

* ``latent_attention``: attention over one cached latent row a token plus one rotated key part that all heads share
  (interleaved rotary pairs), with a learned sink logit a head in the softmax's denominator
  (``kairyu_b200/parts/latent_attention.py``), or
* ``attention``: grouped-query attention with an RMS norm over the whole query and the whole key projection, rotary
  positions on the leading ``rot.dims`` columns of every head (pairs (i, i + dims/2)), one added to the softmax's
  denominator, and a sigmoid output gate (``kairyu_b200/parts/gated_attention.py``).

The feed-forward is dense (``down(g * sigmoid(1.702 g) * (u + 1))`` with ``g = min(gate h, limit)``,
``u = clamp(up h, -limit, limit)``), a mixture of silu experts routed by sigmoid scores whose weights multiply the
experts' INPUTS, with an optional shared expert behind a sigmoid gate of one number a token
(``kairyu_b200/parts/moe.py``), or absent.  ``loop: {start, stop, times}``: layers start .. stop - 1 run ``times`` times in a
row with the same weights and then the rest follow; every pass has a cache of its own, which in the spec is one
``LayerSpec`` named by several ``LayerCall`` entries with different cache slots.  The final norm is a layer norm too.

config.json keys::

    architecture: "Mapalorn"    vocab, width    norm: {eps}    loop?: {start, stop, times}
    layers: [ {type, mixer: {...}, mlp: {...} | null}, ... ]
      latent_attention mixer: heads, dim, rot_dim, vdim, kv_rank, scale, rot: {base, dims}     (dims = rot_dim)
      attention mixer:        heads, kv_heads, dim, vdim, scale, rot: {base, dims}             (dims <= dim)
      mlp: kind: "dense", ff, limit
           kind: "moe", expert: {ff}, router: {experts, top}, shared?: {ff}

Tensors: ``embed``, ``l<i>.norm1`` (+ ``.b``), ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,sink,o}`` or
``l<i>.mix.{q,k,v,q.norm,k.norm,g,o}``, ``l<i>.mlp.{gate,up,down}`` or
``l<i>.mlp.{router,e<n>.{gate,up,down},shared.{gate,up,down,sg}}``, ``final.norm`` (+ ``.b``), ``head`` (matrices stored
[out, in]).  The file names no length limit; the engine needs one to size its rotary tables and takes ``max_positions``
if the file gives it, else ``DEFAULT_MAX_POSITIONS``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from kairyu_b200.config.model_config import ConfigError
from kairyu_b200.parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec

DEFAULT_MAX_POSITIONS = 131072
DENSE_ALPHA = 1.702  # g * sigmoid(DENSE_ALPHA * g) * (u + DENSE_SHIFT) in a dense feed-forward
DENSE_SHIFT = 1.0


@dataclass(frozen=True)
class MapalornLayer:
    kind: str  # "latent_attention" | "attention"
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


@dataclass(frozen=True)
class MapalornConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple[MapalornLayer, ...]
    loop: Optional[tuple[int, int, int]]  # (start, stop, times)
    max_position_embeddings: int
    eos_token_ids: tuple[int, ...] = ()
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    def run_order(self) -> list[int]:
        """Layer indices in the order they run."""
        count = len(self.layers)
        if self.loop is None:
            return list(range(count))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))


def _get(table: Any, key: str, where: str) -> Any:
    if not isinstance(table, Mapping) or key not in table or table[key] is None:
        raise ConfigError(f"config.json: {where} is missing {key!r}")
    return table[key]


def _size(table: Any, key: str, where: str) -> int:
    value = _get(table, key, where)
    if type(value) is not int or value < 1:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= 1, got {value!r}")
    return value


def _real(table: Any, key: str, where: str) -> float:
    value = _get(table, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {value!r}")
    return float(value)


def _parse_rot(mixer: Any, where: str) -> tuple[float, int]:
    rot = _get(mixer, "rot", where)
    dims = _size(rot, "dims", f"{where}.rot")
    if dims % 2:
        raise ConfigError(f"config.json: {where}.rot.dims must be even, got {dims}")
    base = _real(rot, "base", f"{where}.rot")
    if base <= 0.0:
        raise ConfigError(f"config.json: {where}.rot.base must be positive, got {base!r}")
    return base, dims


def _parse_mixer(kind: str, mixer: Any, where: str) -> dict[str, Any]:
    if kind not in ("latent_attention", "attention"):
        raise ConfigError(f"config.json: {where}: unknown layer type {kind!r} (latent_attention, attention)")
    base, dims = _parse_rot(mixer, where)
    parsed = dict(
        heads=_size(mixer, "heads", where), dim=_size(mixer, "dim", where), vdim=_size(mixer, "vdim", where),
        scale=_real(mixer, "scale", where), rot_base=base, rot_dims=dims,
    )
    if kind == "latent_attention":
        parsed.update(kv_rank=_size(mixer, "kv_rank", where), rot_dim=_size(mixer, "rot_dim", where))
        if dims != parsed["rot_dim"]:
            raise ConfigError(f"config.json: {where}.rot.dims={dims} differs from rot_dim={parsed['rot_dim']}: the rotated part turns as a whole")
    else:
        parsed.update(kv_heads=_size(mixer, "kv_heads", where))
        if parsed["heads"] % parsed["kv_heads"]:
            raise ConfigError(f"config.json: {where}: heads={parsed['heads']} is not a multiple of kv_heads={parsed['kv_heads']}")
        if dims > parsed["dim"]:
            raise ConfigError(f"config.json: {where}.rot.dims={dims} of dim={parsed['dim']} columns a head")
    return parsed


def _parse_mlp(mlp: Any, where: str) -> Optional[dict[str, Any]]:
    if mlp is None:
        return None
    kind = _get(mlp, "kind", where)
    if kind == "dense":
        return dict(kind="dense", ff=_size(mlp, "ff", where), limit=_real(mlp, "limit", where))
    if kind != "moe":
        raise ConfigError(f"config.json: {where}: unknown feed-forward kind {kind!r} (dense, moe)")
    router = _get(mlp, "router", where)
    parsed = dict(
        kind="moe", experts=_size(router, "experts", f"{where}.router"), top=_size(router, "top", f"{where}.router"),
        ff=_size(_get(mlp, "expert", where), "ff", f"{where}.expert"),
        shared_ff=_size(mlp["shared"], "ff", f"{where}.shared") if mlp.get("shared") is not None else None,
    )
    if parsed["top"] > parsed["experts"]:
        raise ConfigError(f"config.json: {where}: top={parsed['top']} of {parsed['experts']} experts")
    return parsed


def _parse_loop(loop: Any, count: int) -> Optional[tuple[int, int, int]]:
    if loop is None:
        return None
    values = []
    for key in ("start", "stop", "times"):
        value = _get(loop, key, "loop")
        if type(value) is not int or value < 0:
            raise ConfigError(f"config.json: loop.{key} must be an integer >= 0, got {value!r}")
        values.append(value)
    start, stop, times = values
    if not start <= stop <= count:
        raise ConfigError(f"config.json: loop runs layers {start} .. {stop - 1} of {count}")
    if times < 1 and start != stop:
        raise ConfigError(f"config.json: loop.times must be >= 1, got {times}")
    return (start, stop, times) if start != stop else None


def parse_mapalorn(config: Mapping[str, Any]) -> MapalornConfig:
    entries = _get(config, "layers", "the file")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config.json: layers must be a non-empty list")
    layers = []
    for index, entry in enumerate(entries):
        where = f"layers[{index}]"
        kind = _get(entry, "type", where)
        layers.append(MapalornLayer(kind, _parse_mixer(kind, _get(entry, "mixer", where), f"{where}.mixer"),
                                    _parse_mlp(entry.get("mlp"), f"{where}.mlp")))
    limit = config.get("max_positions", DEFAULT_MAX_POSITIONS)
    if type(limit) is not int or limit < 1:
        raise ConfigError(f"config.json: max_positions must be an integer >= 1, got {limit!r}")
    eos = config.get("eos_token_id")
    return MapalornConfig(
        architecture="Mapalorn",
        vocab_size=_size(config, "vocab", "the file"),
        hidden_size=_size(config, "width", "the file"),
        norm_eps=_real(_get(config, "norm", "the file"), "eps", "norm"),
        layers=tuple(layers),
        loop=_parse_loop(config.get("loop"), len(layers)),
        max_position_embeddings=limit,
        eos_token_ids=(eos,) if type(eos) is int else tuple(eos) if isinstance(eos, list) else (),
        raw=dict(config),
    )


def _layer_spec(index: int, layer: MapalornLayer, config: MapalornConfig) -> LayerSpec:
    prefix = f"l{index}"
    width, eps = config.hidden_size, config.norm_eps
    m = layer.mixer
    # angles are formed in 64-bit and rounded once: every table entry is the correctly rounded cosine or sine
    position = PartSpec("rope", rotary_dim=m["rot_dims"], theta=m["rot_base"], scaling=None,
                        max_positions=config.max_position_embeddings, wide_angles=True)
    if layer.kind == "latent_attention":
        mixer = PartSpec(
            "latent_attention", prefix=f"{prefix}.mix", hidden_size=width, num_heads=m["heads"], head_dim=m["dim"], value_dim=m["vdim"],
            kv_rank=m["kv_rank"], scale=m["scale"], window=None, norm_eps=eps, rot_dim=m["rot_dim"], position=position,
            rotary_interleaved=True, sink=True,
        )
    else:
        mixer = PartSpec(
            "gated_attention", prefix=f"{prefix}.mix", hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
            head_dim=m["dim"], value_dim=m["vdim"], scale=m["scale"], norm_eps=eps, qk_norm="projection", position=position,
            rotary_interleaved=False, sink="zero", gate=True, window=None,
        )
    ffn = None
    if layer.mlp is not None:
        f = layer.mlp
        if f["kind"] == "dense":
            ffn = PartSpec("gated_unit", prefix=f"{prefix}.mlp", hidden_size=width, intermediate_size=f["ff"], limit=f["limit"],
                           alpha=DENSE_ALPHA, shift=DENSE_SHIFT)
        else:
            ffn = PartSpec(
                "moe", prefix=f"{prefix}.mlp", hidden_size=width, intermediate_size=f["ff"], num_experts=f["experts"], top=f["top"],
                routing="scores", score_function="sigmoid", correction=False, weight_on="input", limit=None, alpha=1.0, shift=0.0,
                router_bias=False,
                shared_expert=dict(intermediate_size=f["shared_ff"], gate=True) if f["shared_ff"] is not None else None,
            )
    return LayerSpec(
        prefix=prefix, block="parallel", mixer=mixer, ffn=ffn,
        mixer_norm=PartSpec("layernorm", name=f"{prefix}.norm1", size=width, eps=eps), ffn_norm=None,
    )


def mapalorn_spec(config: MapalornConfig) -> ModelSpec:
    specs = tuple(_layer_spec(index, layer, config) for index, layer in enumerate(config.layers))
    # every run of a layer, a looped one each time, is a call with a cache slot of its own
    schedule = tuple(LayerCall(layer=index, cache_slot=slot) for slot, index in enumerate(config.run_order()))
    width = config.hidden_size
    return ModelSpec(
        embedding=PartSpec("token_embedding", name="embed", vocab_size=config.vocab_size, hidden_size=width),
        layers=specs,
        schedule=schedule,
        final_norm=PartSpec("layernorm", name="final.norm", size=width, eps=config.norm_eps),
        head=PartSpec("linear_head", name="head", vocab_size=config.vocab_size, hidden_size=width, tied_to=None),
        vocab_size=config.vocab_size,
        hidden_size=width,
        max_position_embeddings=config.max_position_embeddings,
    )
