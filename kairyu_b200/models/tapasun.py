"""Tapasun: a decoder whose layers are listed one by one in ``config.json``, each with a norm before AND after
each sub-layer (``x += post1(mixer(pre1(x))); x += post2(ff(pre2(x)))``, ``kairyu_b200/parts/block.py``:
``sandwich_norm``).  Every norm of the stream is an RMS norm with ONE number as its weight.  The embedding is scaled.
The mixer of a layer is

* ``attention``: grouped-query attention with a norm a head on queries and keys (weights of ``dim`` entries shared by
  the heads), rotary positions on the leading ``rot.dims`` columns of every head in interleaved pairs (2i, 2i + 1),
  frequencies scaled as ``rot.scaling`` says, and one added to the softmax's denominator.  With ``kv_from: j`` the layer
  has no key and value tensors and attends over the cache layer j wrote (``kairyu_b200/parts/gated_attention.py``);
* ``parallel``: two mixers on the same input, ``left_scale * left + right_scale * right``
  (``kairyu_b200/parts/side_by_side.py``).  Left: grouped-query attention without a query/key norm, with a learned sink
  logit a head and values that are turned by their position before they are cached, the heads' results turned back by
  the query's.  Right: the gated delta rule with one decay a head and key channel, two-step projections for the decay
  and the gate, and a sigmoid gate (``kairyu_b200/parts/delta_rule.py``);
* ``mamba2``: a selective state-space layer (``kairyu_b200/parts/state_space.py``).

The feed-forward is ``down(silu(gate h) * (up h))`` or absent.  The final norm is one more scalar-weight RMS norm.

config.json keys::

    architecture: "Tapasun"    vocab, width    norm: {eps}    embedding: {scale}
    layers: [ {type, mixer: {...}, mlp: {kind: "dense", ff} | null}, ... ]
      attention mixer: heads, kv_heads, dim, vdim, scale, rot: {base, dims, scaling?}, kv_from?: j
      parallel mixer:  left_scale, right_scale,
                       left:  heads, kv_heads, dim, vdim, scale, rot: {base, dims, scaling?}
                       right: heads, kv_heads, dim, vdim, conv  (+ decay_rank?, gate_rank?: see below)
      mamba2 mixer:    heads, vdim, state, groups, norm_groups, conv
      rot.scaling:     {factor, low, high, original}: frequencies whose wavelength is above original/low are divided by
                       factor, those below original/high kept, those between blended; {factor} alone: all divided by factor

Sizes the file does not name come from the tensors' shapes: the ranks of the delta rule's two-step projections
(``a1``, ``g1``).  Tensors: ``embed``, ``l<i>.norm1``, ``norm1b``, ``norm2``, ``norm2b`` (no dimensions),
``l<i>.mix.{q,k,v,q.norm,k.norm,o}``, ``l<i>.mix.left.{q,k,v,sink,o}``,
``l<i>.mix.right.{q,k,v}`` with ``.conv``, ``l<i>.mix.right.{b,A_log,norm,a1,a2,dt_bias,g1,g2,o}``,
``l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}``, ``l<i>.mlp.{gate,up,down}``, ``final.norm``, ``head`` (matrices
stored [out, in]).  The file names no length limit; the engine needs one to size its rotary tables and takes
``max_positions`` if the file gives it, else ``DEFAULT_MAX_POSITIONS``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from kairyu_b200.config.model_config import ConfigError, RopeScaling
from kairyu_b200.parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec

DEFAULT_MAX_POSITIONS = 131072
DEFAULT_LOW_RANK = 16  # the delta rule's two-step projections, where no checkpoint is at hand to read the rank from


@dataclass(frozen=True)
class TapasunLayer:
    kind: str  # "attention" | "parallel" | "mamba2"
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


@dataclass(frozen=True)
class TapasunConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[TapasunLayer, ...]
    max_position_embeddings: int
    eos_token_ids: tuple[int, ...] = ()
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)


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


def _parse_rot(mixer: Any, where: str, dim: int) -> dict[str, Any]:
    rot = _get(mixer, "rot", where)
    where = f"{where}.rot"
    dims = _size(rot, "dims", where)
    if dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}.dims must be even and at most dim={dim}, got {dims}")
    base = _real(rot, "base", where)
    if base <= 0.0:
        raise ConfigError(f"config.json: {where}.base must be positive, got {base!r}")
    scaling = None
    if isinstance(rot, Mapping) and rot.get("scaling") is not None:
        table = rot["scaling"]
        factor = _real(table, "factor", f"{where}.scaling")
        if factor <= 0.0:
            raise ConfigError(f"config.json: {where}.scaling.factor must be positive, got {factor!r}")
        if any(key in table for key in ("low", "high", "original")):
            low, high = _real(table, "low", f"{where}.scaling"), _real(table, "high", f"{where}.scaling")
            if high == low:
                raise ConfigError(f"config.json: {where}.scaling: low and high must differ")
            scaling = ("llama3", factor, low, high, _size(table, "original", f"{where}.scaling"))
        else:
            scaling = ("linear", factor)
    return dict(rot_base=base, rot_dims=dims, rot_scaling=scaling)


def _parse_attention(mixer: Any, where: str) -> dict[str, Any]:
    parsed = dict(
        heads=_size(mixer, "heads", where), kv_heads=_size(mixer, "kv_heads", where), dim=_size(mixer, "dim", where),
        vdim=_size(mixer, "vdim", where), scale=_real(mixer, "scale", where),
    )
    if parsed["heads"] % parsed["kv_heads"]:
        raise ConfigError(f"config.json: {where}: heads={parsed['heads']} is not a multiple of kv_heads={parsed['kv_heads']}")
    parsed.update(_parse_rot(mixer, where, parsed["dim"]))
    return parsed


def _parse_mixer(kind: str, mixer: Any, where: str) -> dict[str, Any]:
    if kind == "attention":
        parsed = _parse_attention(mixer, where)
        source = mixer.get("kv_from") if isinstance(mixer, Mapping) else None
        if source is not None and (type(source) is not int or source < 0):
            raise ConfigError(f"config.json: {where}.kv_from must name an earlier layer, got {source!r}")
        parsed["kv_from"] = source
        return parsed
    if kind == "parallel":
        left = _parse_attention(_get(mixer, "left", where), f"{where}.left")
        if left["vdim"] % 2:
            raise ConfigError(f"config.json: {where}.left.vdim must be even (the values turn in pairs), got {left['vdim']}")
        r, rw = _get(mixer, "right", where), f"{where}.right"
        right = dict(heads=_size(r, "heads", rw), kv_heads=_size(r, "kv_heads", rw), dim=_size(r, "dim", rw), vdim=_size(r, "vdim", rw),
                     conv=_size(r, "conv", rw),
                     # not keys of the design: a file this package wrote without a checkpoint to read the ranks from may name them
                     decay_rank=_size(r, "decay_rank", rw) if r.get("decay_rank") is not None else None,
                     gate_rank=_size(r, "gate_rank", rw) if r.get("gate_rank") is not None else None)
        if right["heads"] % right["kv_heads"]:
            raise ConfigError(f"config.json: {rw}: heads={right['heads']} is not a multiple of kv_heads={right['kv_heads']}")
        return dict(left=left, right=right, left_scale=_real(mixer, "left_scale", where), right_scale=_real(mixer, "right_scale", where))
    if kind == "mamba2":
        parsed = dict(heads=_size(mixer, "heads", where), vdim=_size(mixer, "vdim", where), state=_size(mixer, "state", where),
                      groups=_size(mixer, "groups", where), norm_groups=_size(mixer, "norm_groups", where), conv=_size(mixer, "conv", where))
        if parsed["heads"] % parsed["groups"]:
            raise ConfigError(f"config.json: {where}: heads={parsed['heads']} is not a multiple of groups={parsed['groups']}")
        if (parsed["heads"] * parsed["vdim"]) % parsed["norm_groups"]:
            raise ConfigError(f"config.json: {where}: heads * vdim = {parsed['heads'] * parsed['vdim']} does not split into norm_groups={parsed['norm_groups']} equal parts")
        return parsed
    raise ConfigError(f"config.json: {where}: unknown layer type {kind!r} (attention, parallel, mamba2)")


def _parse_mlp(mlp: Any, where: str) -> Optional[dict[str, Any]]:
    if mlp is None:
        return None
    kind = _get(mlp, "kind", where)
    if kind != "dense":
        raise ConfigError(f"config.json: {where}: unknown feed-forward kind {kind!r} (dense)")
    return dict(kind="dense", ff=_size(mlp, "ff", where))


def parse_tapasun(config: Mapping[str, Any]) -> TapasunConfig:
    entries = _get(config, "layers", "the file")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config.json: layers must be a non-empty list")
    layers = []
    for index, entry in enumerate(entries):
        where = f"layers[{index}]"
        kind = _get(entry, "type", where)
        layers.append(TapasunLayer(kind, _parse_mixer(kind, _get(entry, "mixer", where), f"{where}.mixer"), _parse_mlp(entry.get("mlp"), f"{where}.mlp")))
    for index, layer in enumerate(layers):
        source = layer.mixer.get("kv_from") if layer.kind == "attention" else None
        if source is None:
            continue
        where = f"layers[{index}].mixer.kv_from"
        if source >= index:
            raise ConfigError(f"config.json: {where}={source} must name an earlier layer")
        other = layers[source]
        if other.kind != "attention" or other.mixer.get("kv_from") is not None:
            raise ConfigError(f"config.json: {where}={source} must name an attention layer with keys and values of its own")
        for key in ("kv_heads", "dim", "vdim"):  # what the borrowed cache's geometry fixes
            if other.mixer[key] != layer.mixer[key]:
                raise ConfigError(f"config.json: {where}={source}: the two layers differ in {key}")
    limit = config.get("max_positions", DEFAULT_MAX_POSITIONS)
    if type(limit) is not int or limit < 1:
        raise ConfigError(f"config.json: max_positions must be an integer >= 1, got {limit!r}")
    eos = config.get("eos_token_id")
    embedding = config.get("embedding")
    return TapasunConfig(
        architecture="Tapasun",
        vocab_size=_size(config, "vocab", "the file"),
        hidden_size=_size(config, "width", "the file"),
        norm_eps=_real(_get(config, "norm", "the file"), "eps", "norm"),
        embedding_scale=_real(embedding, "scale", "embedding") if embedding is not None else 1.0,
        layers=tuple(layers),
        max_position_embeddings=limit,
        eos_token_ids=(eos,) if type(eos) is int else tuple(eos) if isinstance(eos, list) else (),
        raw=dict(config),
    )


def _rope(base: float, dims: int, scaling: Optional[tuple], limit: int) -> PartSpec:
    held = None
    if scaling is not None and scaling[0] == "llama3":
        _, factor, low, high, original = scaling
        held = RopeScaling(kind="llama3", factor=factor, low_freq_factor=low, high_freq_factor=high, original_max_position_embeddings=original)
    elif scaling is not None:
        held = RopeScaling(kind="linear", factor=scaling[1])
    return PartSpec("rope", rotary_dim=dims, theta=base, scaling=held, max_positions=limit, wide_angles=True)


def _attention_spec(prefix: str, m: Mapping[str, Any], config: TapasunConfig, **options: Any) -> PartSpec:
    return PartSpec(
        "gated_attention", prefix=prefix, hidden_size=config.hidden_size, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
        value_dim=m["vdim"], scale=m["scale"], norm_eps=config.norm_eps, rotary_interleaved=True, gate=False,
        position=_rope(m["rot_base"], m["rot_dims"], m["rot_scaling"], config.max_position_embeddings), **options,
    )


def _low_rank(config: TapasunConfig, name: str, named: Optional[int]) -> int:
    """The rank of a two-step projection: the first step's rows, as the checkpoint's header gave them
    (``raw["tensor_shapes"]``, filled in by the loader when it has a file), else what the file names, else the default."""
    shapes = config.raw.get("tensor_shapes") or {}
    shape = shapes.get(name)
    return int(shape[0]) if shape else (named or DEFAULT_LOW_RANK)


def _layer_spec(index: int, layer: TapasunLayer, config: TapasunConfig) -> LayerSpec:
    prefix = f"l{index}"
    width, eps = config.hidden_size, config.norm_eps
    m = layer.mixer
    if layer.kind == "attention":
        mixer = _attention_spec(f"{prefix}.mix", m, config, qk_norm="head", sink="zero", own_kv=m["kv_from"] is None)
    elif layer.kind == "parallel":
        left, right = m["left"], m["right"]
        # the values turn over all their columns, by unscaled frequencies of their own width
        value_position = _rope(left["rot_base"], left["vdim"], None, config.max_position_embeddings)
        mixer = PartSpec(
            "side_by_side", hidden_size=width, left_scale=m["left_scale"], right_scale=m["right_scale"],
            left=_attention_spec(f"{prefix}.mix.left", left, config, qk_norm=None, sink="learned", value_position=value_position),
            right=PartSpec(
                "gated_delta", prefix=f"{prefix}.mix.right", hidden_size=width, num_heads=right["heads"], num_kv_heads=right["kv_heads"],
                head_dim=right["dim"], value_dim=right["vdim"], conv_taps=right["conv"], norm_eps=eps, decay="channel",
                decay_rank=_low_rank(config, f"{prefix}.mix.right.a1", right["decay_rank"]),
                gate_rank=_low_rank(config, f"{prefix}.mix.right.g1", right["gate_rank"]),
                gate_activation="sigmoid",
            ),
        )
    else:
        mixer = PartSpec(
            "state_space_dual", prefix=f"{prefix}.mix", hidden_size=width, num_heads=m["heads"], value_dim=m["vdim"], state_size=m["state"],
            groups=m["groups"], norm_groups=m["norm_groups"], conv_taps=m["conv"], norm_eps=eps,
        )

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", name=f"{prefix}.{name}", size=width, eps=eps, scalar=True)

    ffn = None
    if layer.mlp is not None:
        ffn = PartSpec("swiglu", prefix=f"{prefix}.mlp", hidden_size=width, intermediate_size=layer.mlp["ff"], activation="silu",
                       names=("gate", "up", "down"))
    return LayerSpec(
        prefix=prefix, block="sandwich_norm", mixer=mixer, ffn=ffn, mixer_norm=norm("norm1"), mixer_post_norm=norm("norm1b"),
        ffn_norm=norm("norm2") if ffn is not None else None, ffn_post_norm=norm("norm2b") if ffn is not None else None,
    )


def tapasun_spec(config: TapasunConfig) -> ModelSpec:
    # A layer with keys and values of its own writes the cache slot of its index; a layer with kv_from reads the
    # slot of the layer it names and keeps nothing itself.
    layers = tuple(_layer_spec(index, layer, config) for index, layer in enumerate(config.layers))
    calls = []
    for index, layer in enumerate(config.layers):
        source = layer.mixer.get("kv_from") if layer.kind == "attention" else None
        calls.append(LayerCall(layer=index, cache_slot=index) if source is None else LayerCall(layer=index, cache_slot=source, writes_cache=False))
    width = config.hidden_size
    return ModelSpec(
        embedding=PartSpec("token_embedding", name="embed", vocab_size=config.vocab_size, hidden_size=width, scale=config.embedding_scale),
        layers=layers,
        schedule=tuple(calls),
        final_norm=PartSpec("rmsnorm", name="final.norm", size=width, eps=config.norm_eps, scalar=True),
        head=PartSpec("linear_head", name="head", vocab_size=config.vocab_size, hidden_size=width, tied_to=None),
        vocab_size=config.vocab_size,
        hidden_size=width,
        max_position_embeddings=config.max_position_embeddings,
    )
