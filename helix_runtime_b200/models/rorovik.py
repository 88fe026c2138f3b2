"""The Rorovik decoder as a list of parts.

The token's row of the table passes the model's RMS norm (plain weight); that is the residual's
start.  A layer has a norm on either side of each sublayer and a constant ``m`` on what it adds:
``x += m * norm_b(mixer(norm(x)))``, then the same with the feed-forward (a layer may have none),
then an input of the layer's own that is looked up by the token's id: ``g = gelu_tanh(G x) * e``
with ``e`` the layer's piece of the token's row of a second table, ``y = P g``, ``x += m * y /
rms(y) * w``.  Mixers: ``attention`` (grouped key/value heads, biases, one norm over all of a
token's query coordinates and one over its keys, no rotation, a factor on the query that grows
with the logarithm of the position, a bias on the scores that falls linearly with the distance at
a slope per head, a sliding window, a learned sink in the softmax's denominator, values blended
with the first such layer's, one sigmoid gate per head) and ``latent_attention`` (queries through
a normed latent, one cached latent with a rotated key part shared by the heads, interleaved
rotary pairs whose frequencies are stretched for long contexts, causal, a sink).  The
feed-forward is dense (``down(relu(gate h + b) * (up h + b)) + b``) or a mixture of experts: a
softmax router over the experts and a few outputs that return their input, a correction added
for the choice only, weights that are the chosen scores as they are, and experts with a clamped
gate.  The model ends with the same kind of norm and an untied head.

Tensor names: ``embed``, ``embed.norm``, ``side.embed``; per layer ``l<i>.norm{1,2,1b,2b}``,
``l<i>.mix.{q,k,v}`` with ``.b``, ``l<i>.mix.{q.norm,k.norm,vmix,sink,g,o}`` (attention);
``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,o}`` (latent_attention);
``l<i>.mlp.{gate,up,down}`` with ``.b`` (dense); ``l<i>.mlp.{router,correction}``,
``l<i>.mlp.e<j>.{gate,up,down}`` (experts); ``l<i>.side.{gate,proj,norm}``; ``final.norm``,
``head``.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

from ..config.rorovik import (ARCHITECTURE, CausalLatentAttentionConfig, FeedForwardConfig,
                              RorovikConfig, WindowedAttentionConfig)
from ..config.registry import register_architecture
from ..config.spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry

SLOPE_EXPONENT = 8.0         # head h of H lowers a score by 2^(-8 (h + 1) / H) per position
RESIDUAL_CAST = "rorovik.residual_rows"      # scratch: the residual in the compute type


def distance_slopes(heads: int):
    return tuple(2.0 ** (-SLOPE_EXPONENT * (head + 1) / heads) for head in range(heads))


def _attention(prefix: str, mixer: WindowedAttentionConfig, config: RorovikConfig,
               first_value_mixer: Optional[int], index: int) -> PartSpec:
    roles = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_bias": "q.b", "k_bias": "k.b",
             "v_bias": "v.b", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink",
             "value_mix": "vmix"}
    params = {
        "num_heads": mixer.heads, "num_kv_heads": mixer.kv_heads, "head_dim": mixer.dim,
        "value_dim": mixer.vdim, "scale": mixer.scale, "window": mixer.window, "bias": True,
        "whole_norm": {"eps": config.norm_eps}, "sinks": True,
        "distance_slopes": distance_slopes(mixer.heads), "output_gate": "sigmoid_per_head",
    }
    if mixer.temp_every is not None:
        params["query_temperature"] = {"coef": mixer.temp_coef, "every": mixer.temp_every}
    if mixer.v_mix:
        params["value_mix"] = "source" if index == first_value_mixer else "mix"
    return PartSpec("normed_projection_attention", params,
                    {role: f"{prefix}.mix.{name}" for role, name in roles.items()})


def _latent_attention(prefix: str, mixer: CausalLatentAttentionConfig, config: RorovikConfig,
                      first_value_mixer: Optional[int], index: int) -> PartSpec:
    roles = {"q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "kv_down": "dkv",
             "kv_norm": "dkv.norm", "k_up": "uk", "v_up": "uv", "o": "o", "sink": "sink"}
    rotary = {"theta": mixer.rot_base, "dims": mixer.rot_dims, "layout": "interleaved"}
    if mixer.scaling is not None:
        rotary["scaling"] = {"factor": mixer.scaling.factor, "original": mixer.scaling.original,
                             "fast": mixer.scaling.fast, "slow": mixer.scaling.slow}
    return PartSpec("latent_attention", {
        "num_heads": mixer.heads, "head_dim": mixer.dim, "rotated_dim": mixer.rot_dim,
        "value_dim": mixer.vdim, "kv_rank": mixer.kv_rank, "q_rank": mixer.q_rank,
        "scale": mixer.scale, "window": None, "eps": config.norm_eps, "rotary": rotary,
        "output_gate": None, "sinks": True,
    }, {role: f"{prefix}.mix.{name}" for role, name in roles.items()})


# one builder per value of a layer's ``type``
MIXER_SPECS: Dict[str, Callable[..., PartSpec]] = {
    "attention": _attention, "latent_attention": _latent_attention}


def _feed_forward(prefix: str, mlp: FeedForwardConfig) -> PartSpec:
    if mlp.kind == "dense":
        return PartSpec("gated_mlp", {"intermediate_size": mlp.ff, "activation": "relu",
                                      "bias": True},
                        {"gate": f"{prefix}.mlp.gate", "up": f"{prefix}.mlp.up",
                         "down": f"{prefix}.mlp.down", "gate_bias": f"{prefix}.mlp.gate.b",
                         "up_bias": f"{prefix}.mlp.up.b", "down_bias": f"{prefix}.mlp.down.b"})
    names = {"router": f"{prefix}.mlp.router", "correction": f"{prefix}.mlp.correction"}
    for expert in range(mlp.experts):
        for role in ("gate", "up", "down"):
            names[f"{role}.{expert}"] = f"{prefix}.mlp.e{expert}.{role}"
    return PartSpec("routed_experts", {
        "experts": mlp.experts, "identity": mlp.identity, "top": mlp.top,
        "intermediate_size": mlp.ff, "score": "softmax", "correction": True, "normalize": False,
        "scale": 1.0, "activation": "clamped_sigmoid", "limit": mlp.limit}, names)


def build_rorovik_spec(config: RorovikConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("rms", {"eps": config.norm_eps}, {"weight": name})

    def joined(name: str, cast: bool) -> PartSpec:
        params = {"eps": config.norm_eps, "scale": config.residual_mult}
        if cast:
            params["cast_to"] = RESIDUAL_CAST
        return PartSpec("post_norm", params, {"weight": name})

    value_mixers = [index for index, layer in enumerate(config.layers)
                    if layer.type == "attention" and layer.mixer.v_mix]
    first_value_mixer = value_mixers[0] if value_mixers else None
    side = config.side_dim
    blocks, schedule = [], []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}"
        has_mlp = layer.mlp is not None
        # the sublayer that runs last hands the token input the residual in the compute type
        blocks.append(BlockSpec(
            arrangement="streams",
            mixer_norm=norm(f"{prefix}.norm1"),
            mixer=MIXER_SPECS[layer.type](prefix, layer.mixer, config, first_value_mixer, index),
            feed_forward_norm=norm(f"{prefix}.norm2") if has_mlp else None,
            feed_forward=_feed_forward(prefix, layer.mlp) if has_mlp else None,
            mixer_connection=joined(f"{prefix}.norm1b", side is not None and not has_mlp),
            feed_forward_connection=joined(f"{prefix}.norm2b", side is not None)
            if has_mlp else None,
        ))
        after = None
        if side is not None:
            after = PartSpec("token_side", {
                "dim": side, "offset": index * side, "table_columns": len(config.layers) * side,
                "vocab_size": config.vocab, "eps": config.norm_eps,
                "scale": config.residual_mult, "reads": RESIDUAL_CAST,
            }, {"table": "side.embed", "gate": f"{prefix}.side.gate",
                "proj": f"{prefix}.side.proj", "norm": f"{prefix}.side.norm"})
        schedule.append(ScheduleEntry(block=index, after=after))
    return ModelSpec(
        architecture=config.architecture,
        hidden_size=config.width,
        vocab_size=config.vocab,
        max_positions=config.max_positions,
        embedding=PartSpec("token_table", {"vocab_size": config.vocab, "norm": norm("embed.norm")},
                           {"weight": "embed"}),
        blocks=tuple(blocks),
        schedule=tuple(schedule),
        final_norm=norm("final.norm"),
        lm_head=PartSpec("linear", {"vocab_size": config.vocab, "tied": False}, {"weight": "head"}),
    )


register_architecture(ARCHITECTURE, RorovikConfig.from_dict, build_rorovik_spec,
                      aliases=("rorovik",))
