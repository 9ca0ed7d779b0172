"""``Rabapel``: a decoder whose layers run their mixer and their feed-forward side by side behind ONE
RMS norm (``n = norm(x); x += mixer(n) + ff(n)``).  The mixer is attention over a compressed latent with
directly projected queries, a stretched rotary table on adjacent channel pairs, a sliding window and one
gate number per head; the feed-forward, layer by layer as config.json says, is dense with the squared
rectifier, a mixture of SiLU-gated experts (softmax router, a correction that only steers the choice,
identity experts, a gated shared expert), or absent.  The embedding is scaled by a constant and the head
is the embedding table itself.  Described as data: every part is a registry kind that gets its sizes
and constants as parameters.

Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.mix.q|dkv|dkv.norm|uk|uv|g|o``,
``l<i>.mlp.up|down`` (dense) or ``l<i>.mlp.router|correction|e<j>.gate|up|down|shared.gate|up|down|sg``.
"""
from __future__ import annotations

from typing import Iterator, Tuple

from ..config.rabapel_config import RabapelConfig
from ..config.registry import register_architecture
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleItem

_GATED = {"gate": "gate", "up": "up", "down": "down"}


def build_rabapel_spec(cfg: RabapelConfig) -> ModelSpec:
    H = cfg.width

    def norm(name: str) -> PartSpec:
        i = name.rindex(".") + 1
        return PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "tensor": name[i:]}, prefix=name[:i])

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        mixer = PartSpec("latent_attention", {
            "hidden_size": H, "n_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
            "v_head_dim": m["vdim"], "q_rank": 0, "kv_rank": m["kv_rank"], "softmax_scale": m["scale"],
            "rope_base": m["rot_base"], "rope_scaling": m["rot_scaling"], "rot_dims": m["rot_dims"],
            "pairing": "pairs", "window": m["window"], "eps": cfg.norm_eps, "gate": True, "gate_per_head": True},
            prefix=p + "mix.")
        mlp, ff = layer["mlp"], None
        if mlp is not None and mlp["kind"] == "dense":
            ff = PartSpec("dense_mlp", {"hidden_size": H, "intermediate_size": mlp["ff"], "activation": "relu2",
                                        "names": {"up": "up", "down": "down"}}, prefix=p + "mlp.")
        elif mlp is not None:
            shared = None
            if mlp["shared_ff"]:
                shared = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": mlp["shared_ff"],
                                             "activation": "silu", "names": _GATED}, prefix=p + "mlp.shared.")
            ff = PartSpec("routed_experts", {
                "hidden_size": H, "intermediate_size": mlp["ff"], "n_experts": mlp["experts"],
                "n_identity": mlp["identity"], "top": mlp["top"], "scoring": "softmax", "choice_bias": "correction",
                "alpha": 1.0, "up_offset": 0.0, "limit": None, "shared": shared,
                "shared_gate": "shared.sg" if shared is not None else None}, prefix=p + "mlp.")
        layers.append(LayerSpec(block="parallel_shared_norm", mixer=mixer, mixer_norm=norm(p + "norm1"),
                                feed_forward=ff))
        schedule.append(ScheduleItem(i))
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": H, "tensor": "embed",
                                               "scale": cfg.embedding_scale}),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
        # the head is the embedding table, without the embedding's scale
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": H, "tensor": "embed"}),
    )


def rabapel_random_tensors(cfg: RabapelConfig) -> Iterator[Tuple[str, Tuple[int, ...], object]]:
    """Names, shapes and kinds of a checkpoint of this configuration, in file order."""
    H = cfg.width
    yield "embed", (cfg.vocab, H), "matrix"
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        nh, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        yield p + "norm1", (H,), "norm"
        yield p + "mix.q", (nh * (d + r), H), "matrix"
        yield p + "mix.dkv", (rank + r, H), "matrix"
        yield p + "mix.dkv.norm", (rank,), "norm"
        yield p + "mix.uk", (nh * d, rank), "matrix"
        yield p + "mix.uv", (nh * dv, rank), "matrix"
        yield p + "mix.g", (nh, H), "matrix"
        yield p + "mix.o", (H, nh * dv), "matrix"
        mlp = layer["mlp"]
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            yield p + "mlp.up", (mlp["ff"], H), "matrix"
            yield p + "mlp.down", (H, mlp["ff"]), "matrix"
            continue
        for e in range(mlp["experts"]):
            yield p + f"mlp.e{e}.gate", (mlp["ff"], H), "matrix"
            yield p + f"mlp.e{e}.up", (mlp["ff"], H), "matrix"
            yield p + f"mlp.e{e}.down", (H, mlp["ff"]), "matrix"
        n_out = mlp["experts"] + mlp["identity"]
        yield p + "mlp.router", (n_out, H), "matrix"
        yield p + "mlp.correction", (n_out,), (0.0, 0.01)
        if mlp["shared_ff"]:
            yield p + "mlp.shared.gate", (mlp["shared_ff"], H), "matrix"
            yield p + "mlp.shared.up", (mlp["shared_ff"], H), "matrix"
            yield p + "mlp.shared.down", (H, mlp["shared_ff"]), "matrix"
            yield p + "mlp.shared.sg", (1, H), "matrix"
    yield "final.norm", (H,), "norm"


register_architecture("Rabapel", RabapelConfig, build_rabapel_spec, rabapel_random_tensors, replace=True)
