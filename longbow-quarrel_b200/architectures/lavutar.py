"""The Lavutar decoder, described from parts.

A list of pre-norm layers with layer norms (weight and bias), each with its own mixer and sizes:
"attention" (grouped queries, rotation of a head's first dimensions with YaRN-blended frequencies, a sliding
window, one more 1 in the softmax denominator), "attention_2" (one weighted unit norm over the whole query
projection and one over the key projection, no rotation, capped scores, positions that see their own block of
positions only, a learned term in the denominator, one sigmoid gate per head), or "parallel" (softmax attention
with per-head unit norms of q and k, a query temperature that grows with the position and a sigmoid gate per value,
side by side with gated linear attention whose key channels decay each at its own rate; the two outputs are
added with fixed scales).  The feed-forward is gated with the tanh form of gelu, or routed experts (silu, gated;
the weights are the softmax over the chosen logits).  A stretch of layers may run several times with the same
weights; each pass starts with x <- W_in [x; e], e the embedding's output, and every run of a layer has its own
cache entry.  The head has its own matrix.

Tensor names: `embed`, `loop.in`, `l<i>.norm1 | norm2` with biases `<name>.b`, `l<i>.mix.<q|k|v|o|g|sink|q.norm|k.norm>`
or `l<i>.mix.left.<q|k|v|g|o>` and `l<i>.mix.right.<q|k|v|g|o|norm|a1|a2|a2.b>`, `l<i>.mlp.<gate|up|down>` or
`l<i>.mlp.router`, `l<i>.mlp.e<j>.<gate|up|down>`; `final.norm`, `final.norm.b`, `head`.
"""
from __future__ import annotations

from ..config.lavutar import LavutarConfig, LavutarLayer, SoftmaxHeads
from ..config.registry import register_architecture
from ..parts.rope import YarnScaling
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _norm(cfg: LavutarConfig, name: str) -> PartSpec:
    return PartSpec("layer_norm", {"size": cfg.width, "eps": cfg.norm_eps, "name": name})


def _softmax_attention(cfg: LavutarConfig, a: SoftmaxHeads, kind: str, prefix: str) -> PartSpec:
    params = {"hidden_size": cfg.width, "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "value_dim": a.vdim,
              "scale": a.scale, "names": {k: prefix + k for k in ("q", "k", "v", "o", "g", "sink")}}
    params["names"].update(q_norm=prefix + "q.norm", k_norm=prefix + "k.norm")
    if kind == "attention":
        if a.rot is not None:
            rot = a.rot
            scaling = YarnScaling(rot.factor, rot.original, rot.fast, rot.slow) if rot.factor is not None else None
            params["position"] = PartSpec("rope", {"head_dim": a.dim, "theta": rot.base, "rotary_dims": rot.dims, "scaling": scaling})
        params.update(window=a.span, sink="one")
    elif kind == "attention_2":
        params.update(qk_norm="all", norm_eps=cfg.norm_eps, softcap=a.softcap, chunk=a.span, sink=True, gate="sigmoid_head")
    else:
        params.update(qk_norm="head", norm_eps=cfg.norm_eps, gate="sigmoid",
                      q_temp=(a.temp_coef, a.temp_every) if a.temp_coef is not None else None)
    return PartSpec("attention", params)


def _mixer(cfg: LavutarConfig, layer: LavutarLayer) -> PartSpec:
    if layer.type != "parallel":
        return _softmax_attention(cfg, layer.attn, layer.type, "mix.")
    r = layer.right
    right = PartSpec("channel_decay", {"hidden_size": cfg.width, "n_heads": r.heads, "key_dim": r.dim, "value_dim": r.vdim,
                                       "tau": r.tau, "rank": r.rank, "eps": cfg.norm_eps})
    return PartSpec("side_by_side", {"left": _softmax_attention(cfg, layer.attn, "left", ""), "right": right,
                                     "left_scale": layer.left_scale, "right_scale": layer.right_scale,
                                     "left_prefix": "mix.left.", "right_prefix": "mix.right."})


def _ffn(cfg: LavutarConfig, layer: LavutarLayer) -> PartSpec:
    mlp = layer.mlp
    if mlp.kind == "dense":
        return PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp.ff, "activation": "gelu_tanh",
                                      "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
    return PartSpec("routed_experts", {
        "hidden_size": cfg.width, "n_experts": mlp.experts, "top": mlp.top, "expert_size": mlp.ff, "activation": "silu",
        "gated": True, "score": "softmax", "normalize": True,
        "names": {"router": "mlp.router", "expert": "mlp.e{}", "gate": "gate", "up": "up", "down": "down"}})


def describe(cfg: LavutarConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(cfg.layers):
        parts = dict(norm1=_norm(cfg, "norm1"), mixer=_mixer(cfg, layer))
        if layer.mlp is not None:
            parts.update(norm2=_norm(cfg, "norm2"), ffn=_ffn(cfg, layer))
        layers.append(LayerSpec(prefix=f"l{i}.", arrangement="pre_norm", parts=parts))
    schedule, entry = [], 0
    if cfg.loop is not None:
        layers.append(LayerSpec(prefix="loop.", arrangement="stream_mix", parts={}, params={"hidden_size": cfg.width, "name": "in"}))
    for i, starts_pass in cfg.runs():
        if starts_pass:
            schedule.append(ScheduleEntry(layer=len(cfg.layers), cache=entry))       # it keeps nothing: the entry stays empty
            entry += 1
        schedule.append(ScheduleEntry(layer=i, cache=entry))                          # every run of a layer has its own entry
        entry += 1
    return ModelSpec(
        name="Lavutar", hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed"}),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "head"}),
        max_positions=cfg.max_positions)


register_architecture("Lavutar", LavutarConfig.from_dict, describe)
