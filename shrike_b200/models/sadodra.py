"""Sadodra: a small decoder whose layers are listed one by one in config.json.

    x = embed[token] + pos[position]
    every layer:  x += norm1(mixer(x));  x += norm2(mlp(x))     (layer norms with bias on the branch's
                                                                 OUTPUT; both branches read x itself)
    logits = head . final_norm(x)

`layers[i]` gives `type` (which mixer), `mixer` (its sizes and constants) and `mlp` (null: the layer has
no feed-forward and no second norm).  Mixers:

  attention         heads / kv_heads / dim; the values are the keys as projected (vdim = dim, no value
                    matrix); q and k RMS-normed over the whole projection; `q_temp` {coef, every};
                    `scale`; `softcap`; a distance bias with slope 2^(-8 (h + 1) / heads) for head h;
                    `mask` {size}: a sliding window.  Optional keys that are absent switch their
                    mechanism off.
  latent_attention  heads / dim / vdim / kv_rank; only the RMS-normed latent is cached; causal; an
                    output gate per head; `kv_from`: j makes the layer attend over layer j's latent
                    (it has no down-projection of its own).

Feed-forward: `kind` dense, gated with the tanh form of GELU.  `norm.eps` serves every norm.
Tensor names: `embed`, `pos`, `l<i>.norm1` (+ `.b`), `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`,
`final.norm` (+ `.b`), `head`.
"""

from __future__ import annotations

from ..config.model_config import (
    ConfigError,
    GatedMLPSpec,
    LatentAttentionSpec,
    LayerNormSpec,
    LayerRun,
    LayerSpec,
    LMHeadSpec,
    ModelConfig,
    SharedKeyValueAttentionSpec,
    TokenPositionEmbeddingSpec,
    normalise_dtype,
    require,
)
from ..config.registry import Architecture, TensorNames, register_architecture

SLOPE_DECAY = 8.0   # head h of H takes 2^(-8 (h + 1) / H) per position of distance off its scores


def _mixer_key(layer: dict, index: int, key: str, kind=None):
    mixer = layer.get("mixer")
    if not isinstance(mixer, dict):
        raise ConfigError(f"config.json: layers[{index}] lacks `mixer`")
    try:
        return require(mixer, key, kind)
    except ConfigError as error:
        raise ConfigError(f"layers[{index}].mixer: {error}") from None


def parse_sadodra(raw: dict) -> ModelConfig:
    width = require(raw, "width", int)
    vocab = require(raw, "vocab", int)
    max_positions = require(raw, "max_positions", int)
    listed = require(raw, "layers")
    if not isinstance(listed, list) or not listed:
        raise ConfigError("config.json: `layers` must be a non-empty list")
    eps = float(require(require(raw, "norm"), "eps", float))
    norm = LayerNormSpec(width=width, eps=eps, bias=True)

    layers, order = [], []
    for index, layer in enumerate(listed):
        kind = layer.get("type")
        mixer = layer.get("mixer") or {}
        cache, writes = index, True
        if kind == "attention":
            dim = _mixer_key(layer, index, "dim", int)
            if mixer.get("vdim", dim) != dim:
                raise ConfigError(f"layers[{index}].mixer: the values are the keys, so vdim must equal dim")
            temp = mixer.get("q_temp")
            mask = mixer.get("mask")
            spec = SharedKeyValueAttentionSpec(
                width=width,
                num_heads=_mixer_key(layer, index, "heads", int),
                num_kv_heads=_mixer_key(layer, index, "kv_heads", int),
                head_dim=dim,
                scale=float(_mixer_key(layer, index, "scale", float)),
                eps=eps,
                qk_norm=True,
                q_temperature=None if temp is None else (float(require(temp, "coef", float)), require(temp, "every", int)),
                softcap=None if mixer.get("softcap") is None else float(mixer["softcap"]),
                slope_decay=SLOPE_DECAY,
                window=None if mask is None else require(mask, "size", int),
            )
        elif kind == "latent_attention":
            source = mixer.get("kv_from")
            rank = _mixer_key(layer, index, "kv_rank", int)
            if source is not None:
                if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < index:
                    raise ConfigError(f"layers[{index}].mixer.kv_from must name an earlier layer, got {source!r}")
                theirs = listed[source]
                if theirs.get("type") != "latent_attention" or (theirs.get("mixer") or {}).get("kv_from") is not None:
                    raise ConfigError(f"layers[{index}].mixer.kv_from={source}: that layer caches no latent of its own")
                if theirs["mixer"].get("kv_rank") != rank:
                    raise ConfigError(f"layers[{index}].mixer.kv_rank differs from layer {source}'s, whose latent it reads")
                cache, writes = source, False
            spec = LatentAttentionSpec(
                width=width,
                num_heads=_mixer_key(layer, index, "heads", int),
                head_dim=_mixer_key(layer, index, "dim", int),
                value_dim=_mixer_key(layer, index, "vdim", int),
                latent_rank=rank,
                scale=float(_mixer_key(layer, index, "scale", float)),
                eps=eps,
                own_latent=source is None,
                gated=True,
            )
        else:
            raise ConfigError(f"config.json: layers[{index}].type={kind!r}; known: attention, latent_attention")
        mlp = layer.get("mlp")
        ffn = None
        if mlp is not None:
            if mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"layers[{index}].mlp.kind={mlp.get('kind')!r}; known: dense")
            ffn = GatedMLPSpec(width=width, intermediate=require(mlp, "ff", int), activation="gelu_tanh")
        layers.append(LayerSpec(mixer=spec, mixer_norm=norm, feed_forward=ffn,
                                feed_forward_norm=norm if ffn is not None else None, block="branch_norm"))
        order.append(LayerRun(layer=index, cache=cache, writes_cache=writes))

    eos = raw.get("eos_token_id")
    return ModelConfig(
        architecture="Sadodra",
        hidden_size=width,
        vocab_size=vocab,
        layers=layers,
        order=order,
        final_norm=norm,
        tie_word_embeddings=False,
        max_position_embeddings=max_positions,
        eos_token_ids=list(eos) if isinstance(eos, list) else ([] if eos is None else [int(eos)]),
        dtype=normalise_dtype(raw.get("torch_dtype") or raw.get("dtype") or "bfloat16"),
        raw=dict(raw),
        embedding=TokenPositionEmbeddingSpec(vocab=vocab, width=width, max_positions=max_positions),
        head=LMHeadSpec(width=width, vocab=vocab, tied=False),
    )


_ROLE_PREFIX = {"mixer": "mix.", "mixer_norm": "norm1", "feed_forward": "mlp.", "feed_forward_norm": "norm2"}

# a part's own parameter name -> the last piece of the tensor's name in a Sadodra file
_LOCAL = {
    "mixer": {"q_proj.weight": "q", "k_proj.weight": "k", "q_norm.weight": "q.norm", "k_norm.weight": "k.norm",
              "o_proj.weight": "o", "kv_down.weight": "dkv", "kv_norm.weight": "dkv.norm", "k_up.weight": "uk",
              "v_up.weight": "uv", "gate.weight": "g"},
    "feed_forward": {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"},
    "mixer_norm": {"weight": "", "bias": ".b"},
    "feed_forward_norm": {"weight": "", "bias": ".b"},
    "final_norm": {"weight": "", "bias": ".b"},
    "embedding": {"positions": "pos"},
}


def sadodra_tensor_names(config: ModelConfig) -> TensorNames:
    return TensorNames(
        embedding="embed",
        final_norm_prefix="final.norm",
        lm_head="head",
        layer_part=lambda layer, role: f"l{layer}.{_ROLE_PREFIX[role]}",
        embedding_prefix="",
        head_prefix="head.",
        local_name=lambda role, local: _LOCAL[role][local],
    )


SADODRA = register_architecture(
    Architecture(name="Sadodra", parse_config=parse_sadodra, tensor_names=sadodra_tensor_names)
)
