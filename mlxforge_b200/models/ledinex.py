"""``Ledinex``: a decoder whose sublayers read the residual stream itself through a short causal convolution
and are normalised on their way back (``x += norm(sublayer(x + conv(x)))``, RMS norms with weights stored
around zero).  Its layers are, in an order that config.json gives, two mixers side by side - softmax attention
with whole-projection norms beside a recurrent branch (``parallel``: soft-capped causal attention with rotated
values beside a fixed-decay state; ``parallel_2``: sliding-window attention whose values are its raw keys
beside a generalized delta rule) - or a gated delta rule with one decay per head (``delta``), each followed by
a mixture of squared-rectifier experts with a shared expert, or by nothing.  The embedding is scaled by a
constant; the head is the embedding table, its logits times a constant.  Described as data: every part is
a registry kind that gets its sizes and constants as parameters.

Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.norm1|norm2|canon1|canon2``,
``l<i>.mix.left.q|k|v|o|q.b|k.b|q.norm|k.norm``, ``l<i>.mix.right.*`` (``q|k|v|g|o|norm`` or
``r|k|v|a|a.b|g|w1|w2|w0|norm|o``), ``l<i>.mix.q|k|v|*.conv|b|a|A_log|dt_bias|g|norm|o`` (delta),
``l<i>.mlp.router|e<j>.up|e<j>.down|shared.up|shared.down``.
"""
from __future__ import annotations

from typing import Iterator, Tuple

from ..config.ledinex_config import LedinexConfig
from ..config.registry import register_architecture
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleItem

DEFAULT_DECAY_RANK = 16      # of a configuration that does not name it (random weights)


def _attention(cfg: LedinexConfig, a, prefix: str, kind: str) -> PartSpec:
    own = kind == "parallel"
    return PartSpec("normed_attention", {
        "hidden_size": cfg.width, "n_heads": a["heads"], "n_kv_heads": a["kv_heads"], "head_dim": a["dim"],
        "v_head_dim": a["vdim"], "softmax_scale": a["scale"], "softcap": a["softcap"], "window": a["window"],
        "values": "own" if own else "keys", "bias": not own, "qk_norm": "whole", "eps": cfg.norm_eps,
        "rotary": a["rot"], "rotate_values": own, "out_f32": True}, prefix=prefix)


def _mixer(cfg: LedinexConfig, layer, p: str) -> PartSpec:
    H, m, kind = cfg.width, layer["mixer"], layer["type"]
    if kind == "delta":
        return PartSpec("channel_delta", {
            "hidden_size": H, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "v_head_dim": m["vdim"], "conv": m["conv"], "eps": cfg.norm_eps, "decay_rank": 0, "gate_rank": 0,
            "decay_per_head": True, "gate_act": "silu", "out_f32": True}, prefix=p + "mix.")
    r = m["right"]
    if kind == "parallel":
        right = PartSpec("retention", {
            "hidden_size": H, "n_heads": r["heads"], "head_dim": r["dim"], "v_head_dim": r["vdim"], "rotary_dim": 0,
            "key_scale": 1.0, "decay": r["decay"], "eps": cfg.norm_eps, "activation": "silu", "output_norm": "whole",
            "norm_weight": "norm", "gate_act": "sigmoid", "out_f32": True}, prefix=p + "mix.right.")
    else:
        right = PartSpec("generalized_delta", {
            "hidden_size": H, "n_heads": r["heads"], "head_dim": r["dim"],
            "decay_rank": r.get("decay_rank") or DEFAULT_DECAY_RANK, "eps": cfg.norm_eps, "out_f32": True},
            prefix=p + "mix.right.")
    return PartSpec("side_by_side", {"left": _attention(cfg, m["left"], p + "mix.left.", kind), "right": right,
                                     "left_scale": m["left_scale"], "right_scale": m["right_scale"]}, prefix=p + "mix.")


def build_ledinex_spec(cfg: LedinexConfig) -> ModelSpec:
    H = cfg.width

    def norm(name: str, scale: float = 1.0) -> PartSpec:
        i = name.rindex(".") + 1
        return PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "tensor": name[i:], "one_plus": True,
                                    "scale": scale}, prefix=name[:i])

    def conv(name: str) -> PartSpec:
        i = name.rindex(".") + 1
        return PartSpec("conv_read", {"size": H, "taps": cfg.taps, "tensor": name[i:]}, prefix=name[:i])

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        mlp, ff = layer["mlp"], None
        extra = [("mixer_connection", "connection", conv(p + "canon1"))]
        if mlp is not None:
            shared = None
            if mlp["shared_ff"]:
                shared = PartSpec("dense_mlp", {"hidden_size": H, "intermediate_size": mlp["shared_ff"],
                                                "activation": "relu2"}, prefix=p + "mlp.shared.")
            ff = PartSpec("routed_experts", {
                "hidden_size": H, "intermediate_size": mlp["ff"], "n_experts": mlp["experts"], "top": mlp["top"],
                "scoring": "softmax", "renormalize": True, "expert_act": "relu2", "shared": shared},
                prefix=p + "mlp.")
            extra.append(("feed_forward_connection", "connection", conv(p + "canon2")))
        layers.append(LayerSpec(block="postnorm_conv", mixer=_mixer(cfg, layer, p), mixer_norm=norm(p + "norm1"),
                                feed_forward=ff, feed_forward_norm=norm(p + "norm2") if ff is not None else None,
                                extra=tuple(extra)))
        schedule.append(ScheduleItem(i))
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": H, "tensor": "embed",
                                               "scale": cfg.embedding_scale}),
        layers=tuple(layers), schedule=tuple(schedule),
        # the logits' constant multiplies the final norm's rows: E (c n) = c (E n)
        final_norm=norm("final.norm", cfg.logit_scale),
        # the head is the embedding table, without the embedding's scale
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": H, "tensor": "embed"}),
    )


def ledinex_random_tensors(cfg: LedinexConfig) -> Iterator[Tuple[str, Tuple[int, ...], object]]:
    """Names, shapes and kinds of a checkpoint of this configuration, in file order."""
    H = cfg.width
    yield "embed", (cfg.vocab, H), "matrix"
    for i, layer in enumerate(cfg.layers):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        yield p + "norm1", (H,), (0.0, 0.1)
        if cfg.taps:
            yield p + "canon1", (H, cfg.taps), (0.0, 0.2)
        if kind == "delta":
            nqk, nv, nh = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m["heads"]
            for r, n in (("q", nqk), ("k", nqk), ("v", nv)):
                yield p + "mix." + r, (n, H), "matrix"
                yield p + "mix." + r + ".conv", (n, m["conv"]), (0.0, 0.5)
            yield p + "mix.b", (nh, H), "matrix"
            yield p + "mix.a", (nh, H), "matrix"
            yield p + "mix.A_log", (nh,), (0.0, 0.5)
            yield p + "mix.dt_bias", (nh,), (0.0, 0.5)
            yield p + "mix.g", (nv, H), "matrix"
            yield p + "mix.norm", (m["vdim"],), "norm"
            yield p + "mix.o", (H, nv), "matrix"
        else:
            a, r = m["left"], m["right"]
            nq, nk, nv = a["heads"] * a["dim"], a["kv_heads"] * a["dim"], a["kv_heads"] * a["vdim"]
            q = p + "mix.left."
            yield q + "q", (nq, H), "matrix"
            yield q + "k", (nk, H), "matrix"
            if kind == "parallel":
                yield q + "v", (nv, H), "matrix"
            else:
                yield q + "q.b", (nq,), (0.0, 0.1)
                yield q + "k.b", (nk,), (0.0, 0.1)
            yield q + "q.norm", (nq,), "norm"
            yield q + "k.norm", (nk,), "norm"
            yield q + "o", (H, a["heads"] * a["vdim"]), "matrix"
            q = p + "mix.right."
            n = r["heads"] * r["dim"]
            if kind == "parallel":
                nv = r["heads"] * r["vdim"]
                yield q + "q", (n, H), "matrix"
                yield q + "k", (n, H), "matrix"
                yield q + "v", (nv, H), "matrix"
                yield q + "g", (nv, H), "matrix"
                yield q + "norm", (nv,), "norm"
                yield q + "o", (H, nv), "matrix"
            else:
                rank = r.get("decay_rank") or DEFAULT_DECAY_RANK
                for t in ("r", "k", "v", "a", "g"):
                    yield q + t, (n, H), "matrix"
                yield q + "a.b", (n,), (0.0, 0.5)
                yield q + "w1", (rank, H), "matrix"
                yield q + "w2", (n, rank), "matrix"
                yield q + "w0", (n,), (0.0, 0.5)
                yield q + "norm", (n,), "norm"
                yield q + "o", (H, n), "matrix"
        mlp = layer["mlp"]
        if mlp is None:
            continue
        yield p + "norm2", (H,), (0.0, 0.1)
        if cfg.taps:
            yield p + "canon2", (H, cfg.taps), (0.0, 0.2)
        yield p + "mlp.router", (mlp["experts"], H), "matrix"
        for e in range(mlp["experts"]):
            yield p + f"mlp.e{e}.up", (mlp["ff"], H), "matrix"
            yield p + f"mlp.e{e}.down", (H, mlp["ff"]), "matrix"
        if mlp["shared_ff"]:
            yield p + "mlp.shared.up", (mlp["shared_ff"], H), "matrix"
            yield p + "mlp.shared.down", (H, mlp["shared_ff"]), "matrix"
    yield "final.norm", (H,), (0.0, 0.1)


register_architecture("Ledinex", LedinexConfig, build_ledinex_spec, ledinex_random_tensors, replace=True)
