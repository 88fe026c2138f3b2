"""The Medolorn decoder as a list of parts.

The token's row of the table passes the model's norm (``1 + w``); that is the embedding's
output ``x0``.  A layer is pre-norm with gated residuals: ``h = norm(x)``, ``x += sigmoid(G h +
b) * f(h)`` for the mixer and then for the feed-forward, and the mixer reads ``h + conv(h)``,
a causal per-channel filter over time.  Mixers: ``delta`` (linear attention with the gated
delta rule: filtered, unit-length queries and keys, a learned decay and write strength per
head), ``latent_attention`` (sliding-window softmax attention whose keys and values are
up-projections of one cached latent, with a rotated part shared by the heads and a sigmoid
output gate) and ``retention`` (linear attention with a constant decay per head and rotated
queries and keys).  The feed-forward is a mixture of routed experts.  A stretch of layers may
run several times with the same weights (``loop``); every run owns its cache and state, and
before each pass ``x <- W [x ; x0] + step[pass]``.  The model ends with the same kind of norm
and an untied head.

Tensor names: ``embed``, ``embed.norm``, ``loop.in``, ``loop.step``; per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.canon1``, ``l<i>.rg{1,2}``, ``l<i>.rg{1,2}.b``; ``l<i>.mix.{q,k,v,q.conv,
k.conv,v.conv,b,a,A_log,dt_bias,norm,g,o}`` (delta); ``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,
uv,g,o}`` (latent_attention); ``l<i>.mix.{q,k,v,g,o}`` (retention); ``l<i>.mlp.router``,
``l<i>.mlp.e<j>.{gate,up,down}``; ``final.norm``, ``head``.
"""
from __future__ import annotations

from typing import Callable, Dict

from ..config.medolorn import (ARCHITECTURE, DeltaMixerConfig, LatentAttentionConfig,
                               MedolornConfig, RetentionMixerConfig)
from ..config.registry import register_architecture
from ..config.spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry

DELTA_UNIT_EPS = 1e-6        # inside the root that makes queries and keys unit vectors


def _delta_mixer(prefix: str, mixer: DeltaMixerConfig, config: MedolornConfig) -> PartSpec:
    roles = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "beta": "b", "decay": "a",
             "a_log": "A_log", "dt_bias": "dt_bias", "norm": "norm", "q_filter": "q.conv",
             "k_filter": "k.conv", "v_filter": "v.conv"}
    return PartSpec("linear_state", {
        "heads": mixer.heads, "qk_heads": mixer.kv_heads, "head_dim": mixer.dim,
        "value_dim": mixer.vdim, "rule": "delta", "filter_taps": mixer.conv, "unit_norm": True,
        "unit_eps": DELTA_UNIT_EPS, "q_scale": float(mixer.dim) ** -0.5, "norm_weight": True,
        "eps": config.norm_eps,
    }, {role: f"{prefix}.mix.{name}" for role, name in roles.items()})


def _latent_attention(prefix: str, mixer: LatentAttentionConfig, config: MedolornConfig) -> PartSpec:
    roles = {"q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "kv_down": "dkv",
             "kv_norm": "dkv.norm", "k_up": "uk", "v_up": "uv", "g": "g", "o": "o"}
    return PartSpec("latent_attention", {
        "num_heads": mixer.heads, "head_dim": mixer.dim, "rotated_dim": mixer.rot_dim,
        "value_dim": mixer.vdim, "kv_rank": mixer.kv_rank, "q_rank": mixer.q_rank,
        "scale": mixer.scale, "window": mixer.window, "eps": config.norm_eps,
        "rotary": {"theta": mixer.rot_base, "dims": mixer.rot_dims, "layout": "interleaved"},
        "output_gate": "sigmoid",
    }, {role: f"{prefix}.mix.{name}" for role, name in roles.items()})


def _retention_mixer(prefix: str, mixer: RetentionMixerConfig, config: MedolornConfig) -> PartSpec:
    return PartSpec("linear_state", {
        "heads": mixer.heads, "head_dim": mixer.dim, "value_dim": mixer.vdim, "rule": "decay",
        "decay": tuple(mixer.decay), "k_scale": float(mixer.dim) ** -0.5,
        "rotary": {"theta": mixer.rot_base, "dims": mixer.rot_dims, "layout": "halves"},
        "eps": config.norm_eps,
    }, {name: f"{prefix}.mix.{name}" for name in ("q", "k", "v", "g", "o")})


# one builder per value of a layer's ``type``
MIXER_SPECS: Dict[str, Callable[[str, object, MedolornConfig], PartSpec]] = {
    "delta": _delta_mixer, "latent_attention": _latent_attention, "retention": _retention_mixer}


def build_medolorn_spec(config: MedolornConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("rms", {"eps": config.norm_eps, "one_plus": True}, {"weight": name})

    def gate(prefix: str, which: int) -> PartSpec:
        return PartSpec("gated", {}, {"gate": f"{prefix}.rg{which}",
                                      "gate_bias": f"{prefix}.rg{which}.b"})

    blocks = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}"
        mixer = PartSpec("input_filter", {
            "taps": config.canon_taps,
            "mixer": MIXER_SPECS[layer.type](prefix, layer.mixer, config),
        }, {"filter": f"{prefix}.canon1"})
        feed_forward = feed_forward_norm = feed_forward_connection = None
        if layer.mlp is not None:
            names = {"router": f"{prefix}.mlp.router"}
            for expert in range(layer.mlp.experts):
                for role in ("gate", "up", "down"):
                    names[f"{role}.{expert}"] = f"{prefix}.mlp.e{expert}.{role}"
            feed_forward = PartSpec("routed_experts", {
                "experts": layer.mlp.experts, "top": layer.mlp.top,
                "intermediate_size": layer.mlp.ff, "scale": layer.mlp.scale,
                "activation": "silu"}, names)
            feed_forward_norm = norm(f"{prefix}.norm2")
            feed_forward_connection = gate(prefix, 2)
        blocks.append(BlockSpec(
            arrangement="streams",
            mixer_norm=norm(f"{prefix}.norm1"),
            mixer=mixer,
            feed_forward_norm=feed_forward_norm,
            feed_forward=feed_forward,
            mixer_connection=gate(prefix, 1),
            feed_forward_connection=feed_forward_connection,
        ))
    schedule = []
    for layer, starts in config.layer_runs():
        before = None
        if starts is not None:
            before = PartSpec("linear_rejoin", {"index": starts, "steps": config.loop.times},
                              {"weight": "loop.in", "step": "loop.step"})
        schedule.append(ScheduleEntry(block=layer, before=before))
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


register_architecture(ARCHITECTURE, MedolornConfig.from_dict, build_medolorn_spec,
                      aliases=("medolorn",))
