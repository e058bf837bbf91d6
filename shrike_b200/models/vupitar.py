"""Vupitar: a small decoder whose layers are listed one by one in config.json, with a stretch of
layers that runs several times.

    e = embed[token] * embedding.scale
    layers `loop.start` .. `loop.stop` - 1 run `loop.times` times in a row with the same weights and a
    cache and state of their own each pass, then the rest follow.  Entering pass t: x += e (t > 0),
    x += loop.step[t].
    every layer:  x += mixer(N1(x)) + ff(N2(x)),  N(x) = tanh(alpha x) * w + b
    logits = head . N_final(x)

`layers[i]` gives `type` (which mixer), `mixer` (its sizes and constants) and `mlp` (null: none).

  parallel   two mixers that read the same input, added as left_scale * left + right_scale * right:
             `left`  grouped-query softmax attention (heads / kv_heads / dim / vdim) with biases, a
                     root-mean-square norm of q and k per head, `rot` {dims, base}: a rotation of each
                     head's first dims, `scale`, `mask` {size}: positions in runs of that size, a query
                     sees its own run only, and a sigmoid gate per head on the output;
             `right` a matrix memory (heads / dim / vdim / gate_cap), see `parts/matrix_memory.py`.

Feed-forward: `kind` dense (gate clamped from above and up clamped on both sides at `limit`, then
g sigmoid(1.702 g) (u + 1)) or moe (`router` {experts, top}, `expert` {ff}, `shared` {ff}: SiLU-gated
experts, softmax router, a gated shared expert).  `norm.eps` serves the root-mean-square norms inside
the mixers.  Tensor names: `embed`, `loop.step`, `l<i>.norm1` (+ `.b`, `.alpha`), `l<i>.norm2`,
`l<i>.mix.left.*`, `l<i>.mix.right.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""

from __future__ import annotations

from ..config.model_config import (
    ConfigError,
    DynamicTanhSpec,
    GatedHeadAttentionSpec,
    GatedMLPSpec,
    LayerRun,
    LayerSpec,
    LMHeadSpec,
    MatrixMemorySpec,
    ModelConfig,
    ParallelMixerSpec,
    PassEntrySpec,
    RoutedExpertsSpec,
    TokenEmbeddingSpec,
    normalise_dtype,
    require,
)
from ..config.registry import Architecture, TensorNames, register_architecture

DENOMINATOR_FLOOR = 1e-6    # added to the matrix memory's denominator
ROUTER_RENORM_EPS = 1e-20   # added to the sum of the chosen experts' scores
DEFAULT_MAX_POSITIONS = 1 << 20   # the design has no position table: nothing bounds a sequence but the pool


def _sub(raw: dict, key: str, where: str) -> dict:
    value = raw.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where} lacks `{key}`")
    return value


def _need(raw: dict, key: str, kind, where: str):
    try:
        return require(raw, key, kind)
    except ConfigError as error:
        raise ConfigError(f"{where}: {error}") from None


def _left(raw: dict, width: int, eps: float, where: str) -> GatedHeadAttentionSpec:
    dim = _need(raw, "dim", int, where)
    rot, mask = raw.get("rot"), raw.get("mask")
    return GatedHeadAttentionSpec(
        width=width,
        num_heads=_need(raw, "heads", int, where),
        num_kv_heads=_need(raw, "kv_heads", int, where),
        head_dim=dim,
        value_dim=raw.get("vdim", dim) if raw.get("vdim") is not None else dim,
        scale=float(_need(raw, "scale", float, where)),
        eps=eps,
        qkv_bias=True,
        out_bias=True,
        qk_norm=True,
        rotary=None if rot is None else (_need(rot, "dims", int, where + ".rot"), float(_need(rot, "base", float, where + ".rot"))),
        chunk=None if mask is None else _need(mask, "size", int, where + ".mask"),
        head_gate=True,
    )


def _right(raw: dict, width: int, eps: float, where: str) -> MatrixMemorySpec:
    dim = _need(raw, "dim", int, where)
    return MatrixMemorySpec(
        width=width,
        num_heads=_need(raw, "heads", int, where),
        head_dim=dim,
        value_dim=raw.get("vdim", dim) if raw.get("vdim") is not None else dim,
        gate_cap=float(_need(raw, "gate_cap", float, where)),
        eps=eps,
        denominator_floor=DENOMINATOR_FLOOR,
    )


def _feed_forward(mlp: dict, width: int, where: str):
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return GatedMLPSpec(width=width, intermediate=_need(mlp, "ff", int, where), activation="clamped_swish",
                            limit=float(_need(mlp, "limit", float, where)))
    if kind == "moe":
        router = _sub(mlp, "router", where)
        shared = mlp.get("shared")
        return RoutedExpertsSpec(
            width=width,
            experts=_need(router, "experts", int, where + ".router"),
            top=_need(router, "top", int, where + ".router"),
            intermediate=_need(_sub(mlp, "expert", where), "ff", int, where + ".expert"),
            activation="silu",
            shared_intermediate=None if shared is None else _need(shared, "ff", int, where + ".shared"),
            shared_gate=True,
            renorm_eps=ROUTER_RENORM_EPS,
        )
    raise ConfigError(f"{where}.kind={kind!r}; known: dense, moe")


def run_order(count: int, loop: dict | None) -> list[LayerRun]:
    """Every run of a layer in order, each with a cache of its own; the first run of pass t carries `enter=t`."""
    if loop is None:
        return [LayerRun(layer=i, cache=i) for i in range(count)]
    start, stop, times = loop.get("start"), loop.get("stop"), require(loop, "times", int)
    for name, value in (("start", start), ("stop", stop)):
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"config.json: loop.{name} must be an integer, got {value!r}")
    if not 0 <= start < stop <= count:
        raise ConfigError(f"config.json: loop runs layers {start} .. {stop} - 1 of {count}")
    layers = list(range(start))
    enters = [None] * start
    for number in range(times):
        layers += range(start, stop)
        enters += [number] + [None] * (stop - start - 1)
    layers += range(stop, count)
    enters += [None] * (count - stop)
    return [LayerRun(layer=layer, cache=cache, enter=enter) for cache, (layer, enter) in enumerate(zip(layers, enters))]


def parse_vupitar(raw: dict) -> ModelConfig:
    width = require(raw, "width", int)
    vocab = require(raw, "vocab", int)
    listed = require(raw, "layers")
    if not isinstance(listed, list) or not listed:
        raise ConfigError("config.json: `layers` must be a non-empty list")
    eps = float(require(require(raw, "norm"), "eps", float))
    norm = DynamicTanhSpec(width=width)
    layers = []
    for index, layer in enumerate(listed):
        where = f"layers[{index}]"
        kind = layer.get("type")
        if kind != "parallel":
            raise ConfigError(f"config.json: {where}.type={kind!r}; known: parallel")
        mixer = _sub(layer, "mixer", where)
        spec = ParallelMixerSpec(width=width, branches=(
            ("left", _left(_sub(mixer, "left", where + ".mixer"), width, eps, where + ".mixer.left"),
             float(_need(mixer, "left_scale", float, where + ".mixer"))),
            ("right", _right(_sub(mixer, "right", where + ".mixer"), width, eps, where + ".mixer.right"),
             float(_need(mixer, "right_scale", float, where + ".mixer"))),
        ))
        mlp = layer.get("mlp")
        ffn = None if mlp is None else _feed_forward(mlp, width, where + ".mlp")
        layers.append(LayerSpec(mixer=spec, mixer_norm=norm, feed_forward=ffn,
                                feed_forward_norm=norm if ffn is not None else None, block="parallel"))
    loop = raw.get("loop")
    order = run_order(len(layers), loop)
    embedding = raw.get("embedding") or {}
    eos = raw.get("eos_token_id")
    return ModelConfig(
        architecture="Vupitar",
        hidden_size=width,
        vocab_size=vocab,
        layers=layers,
        order=order,
        final_norm=norm,
        tie_word_embeddings=False,
        max_position_embeddings=int(raw.get("max_positions") or DEFAULT_MAX_POSITIONS),
        eos_token_ids=list(eos) if isinstance(eos, list) else ([] if eos is None else [int(eos)]),
        dtype=normalise_dtype(raw.get("torch_dtype") or raw.get("dtype") or "bfloat16"),
        raw=dict(raw),
        embedding=TokenEmbeddingSpec(vocab=vocab, width=width, scale=float(embedding.get("scale", 1.0))),
        head=LMHeadSpec(width=width, vocab=vocab, tied=False),
        pass_entry=None if loop is None else PassEntrySpec(width=width, passes=require(loop, "times", int), add_embedding=True),
    )


_ROLE_PREFIX = {"mixer": "mix.", "mixer_norm": "norm1", "feed_forward": "mlp.", "feed_forward_norm": "norm2"}
_NORM = {"weight": "", "bias": ".b", "alpha": ".alpha"}
_PROJECTIONS = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}
_LEFT = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o", "q_proj.bias": "q.b",
         "k_proj.bias": "k.b", "v_proj.bias": "v.b", "o_proj.bias": "o.b", "q_norm.weight": "q.norm",
         "k_norm.weight": "k.norm", "gate.weight": "g"}
_RIGHT = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "gate.weight": "g", "o_proj.weight": "o",
          "norm.weight": "norm", "input_gate.weight": "i", "input_gate.bias": "i.b", "forget_gate.weight": "f",
          "forget_gate.bias": "f.b"}


def _local(role: str, local: str) -> str:
    """A part's own parameter name -> the last piece of the tensor's name in a Vupitar file."""
    if role in ("mixer_norm", "feed_forward_norm", "final_norm"):
        return _NORM[local]
    if role == "mixer":
        branch, _, rest = local.partition(".")
        return f"{branch}." + (_LEFT if branch == "left" else _RIGHT)[rest]
    if role == "feed_forward":
        if local in _PROJECTIONS:
            return _PROJECTIONS[local]
        if local == "router.weight":
            return "router"
        if local == "shared_gate.weight":
            return "shared.sg"
        prefix, _, rest = local.rpartition(".")          # experts.<e>.gate_proj | shared.gate_proj, then "weight"
        owner, _, projection = prefix.rpartition(".")
        owner = "shared" if owner == "shared" else "e" + owner.split(".")[1]
        return f"{owner}.{_PROJECTIONS[projection + '.' + rest]}"
    if role == "pass_entry":
        return {"step": "loop.step"}[local]
    raise KeyError((role, local))


def vupitar_tensor_names(config: ModelConfig) -> TensorNames:
    return TensorNames(
        embedding="embed",
        final_norm_prefix="final.norm",
        lm_head="head",
        layer_part=lambda layer, role: f"l{layer}.{_ROLE_PREFIX[role]}",
        embedding_prefix="",
        head_prefix="head.",
        pass_entry_prefix="",
        local_name=_local,
    )


VUPITAR = register_architecture(
    Architecture(name="Vupitar", parse_config=parse_vupitar, tensor_names=vupitar_tensor_names)
)
