"""The Raritar decoder, described from parts.

The embedding adds a second table's row chosen by hashing the pair (token before, token).  Every layer is
pre-norm with one multiplier on both branches, norms whose gain is a single number, and a short causal
convolution over time on what the mixer reads.  The mixer is grouped-query attention: interleaved rotary pairs on a part of
each head with frequencies rescaled by wavelength, values divided by their root mean square before they are
cached, scores times a given scale and capped by tanh, a sliding window that keeps a sequence's first positions, and
optionally another layer's keys and values in place of its own.  The feed-forward routes tokens to gated experts
(softmax scores, a correction that counts for the choice only, groups scored by their best member, identity
experts, weights not renormalised) beside a gated shared expert behind a scalar sigmoid gate.  The head has its own matrix.

Tensor names: `embed`, `bigram`, `l<i>.norm1 | norm2 | canon1`, `l<i>.mix.<q|k|v|o>`,
`l<i>.mlp.router | correction`, `l<i>.mlp.e<j>.<gate|up|down>`, `l<i>.mlp.shared.<gate|up|down|sg>`,
`final.norm`, `head`.
"""
from __future__ import annotations

from ..config.raritar import RaritarConfig, RaritarLayer
from ..config.registry import register_architecture
from ..parts.rope import WavelengthScaling
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _norm(cfg: RaritarConfig, name: str) -> PartSpec:
    return PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps, "name": name, "scalar": True})


def _kept(cfg: RaritarConfig, i: int) -> tuple[int | None, int]:
    """What layer i's cache entry must keep: the furthest that the layer itself or any layer that reads its keys
    and values sees (a window, or None for everything; and how many first positions stay)."""
    readers = [cfg.layers[i]] + [layer for layer in cfg.layers if layer.kv_from == i]
    if any(layer.window is None for layer in readers):
        return None, 0
    return max(layer.window for layer in readers), max(layer.keep_first for layer in readers)


def _mixer(cfg: RaritarConfig, i: int, layer: RaritarLayer) -> PartSpec:
    position = None
    if layer.rot is not None:
        rot = layer.rot
        scaling = WavelengthScaling(rot.factor, rot.low, rot.high, rot.original) if rot.factor is not None else None
        position = PartSpec("rope", {"head_dim": layer.dim, "theta": rot.base, "rotary_dims": rot.dims, "scaling": scaling,
                                     "layout": "interleaved"})
    window, keep_first = _kept(cfg, i if layer.kv_from is None else layer.kv_from)
    return PartSpec("attention", {
        "hidden_size": cfg.width, "n_heads": layer.heads, "n_kv_heads": layer.kv_heads, "head_dim": layer.dim,
        "value_dim": layer.vdim, "scale": layer.scale, "position": position, "window": layer.window,
        "keep_first": layer.keep_first, "softcap": layer.softcap, "value_norm_eps": cfg.norm_eps,
        "own_kv": layer.kv_from is None, "cache_window": window, "cache_keep_first": keep_first,
        "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o"}})


def _ffn(cfg: RaritarConfig, layer: RaritarLayer) -> PartSpec:
    mlp, r = layer.mlp, layer.mlp.router
    return PartSpec("routed_experts", {
        "hidden_size": cfg.width, "n_experts": r.experts, "identity": r.identity, "top": r.top, "expert_size": mlp.ff,
        "activation": "silu", "gated": True, "score": "softmax", "correction": True, "group_rule": "max", "normalize": False,
        "groups": r.groups, "keep_groups": r.keep, "shared_size": mlp.shared_ff,
        "names": {"router": "mlp.router", "correction": "mlp.correction", "expert": "mlp.e{}", "gate": "gate", "up": "up",
                  "down": "down", "shared": "mlp.shared", "shared_gate": "mlp.shared.sg"}})


def describe(cfg: RaritarConfig) -> ModelSpec:
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        parts = dict(norm1=_norm(cfg, "norm1"), mixer=_mixer(cfg, i, layer))
        if cfg.taps is not None:
            parts["conv1"] = PartSpec("causal_conv", {"channels": cfg.width, "taps": cfg.taps, "name": "canon1"})
        if layer.mlp is not None:
            parts.update(norm2=_norm(cfg, "norm2"), ffn=_ffn(cfg, layer))
        layers.append(LayerSpec(prefix=f"l{i}.", arrangement="pre_norm", parts=parts,
                                params={"residual_scale": cfg.residual_mult}))
        schedule.append(ScheduleEntry(layer=i, cache=i if layer.kv_from is None else layer.kv_from,
                                      writes_cache=layer.kv_from is None))
    if cfg.bigram is not None:
        embedding = PartSpec("pair_hash_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed",
                                                     "pairs_name": "bigram", "buckets": cfg.bigram.buckets,
                                                     "mul_prev": cfg.bigram.mul_prev, "mul_cur": cfg.bigram.mul_cur})
    else:
        embedding = PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed"})
    return ModelSpec(
        name="Raritar", hidden_size=cfg.width, vocab_size=cfg.vocab, embedding=embedding,
        layers=tuple(layers), schedule=tuple(schedule), final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "head"}),
        max_positions=cfg.max_positions)


register_architecture("Raritar", RaritarConfig.from_dict, describe)
