"""Puledra as a ``ModelSpec``.

Every layer is a parallel block, x <- x + (mixer(n) + ff(n)) with n = rmsnorm(x): the mixer is latent
attention (``parts/latent_attention.py``) with an interleaved rotary encoding on the rotated part, the
feed-forward a mixture of SiLU-gated experts with a softmax router limited to groups
(``grouped_topk_moe``), or absent.  The embedding is the token's row times a constant plus a hashed
row for the pair (previous token, token).  A layer that names another in ``kv_from`` reads that layer's
cached latent (``LayerCall.cache_of``) and has no down-projection of its own.  Checkpoints name tensors
``embed``, ``bigram``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm`` and ``head``.
The reference registers its families in one table keyed by the checkpoint's architecture string
(crates/thuban_architectures/src/loader.rs:39-60).
"""
from __future__ import annotations

from ..config.puledra import DEFAULT_MAX_POSITIONS, PuledraConfig
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..registry import ARCHITECTURES


@ARCHITECTURES.register("Puledra")
class PuledraArchitecture:
    config_class = PuledraConfig

    @staticmethod
    def parse_config(d: dict) -> PuledraConfig:
        return PuledraConfig.from_dict(d)

    @staticmethod
    def model_spec(cfg: PuledraConfig) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.eps})
        layers, order, stored = [], [], {}
        for i, layer in enumerate(cfg.layers):
            m = layer.mixer
            position = PartSpec("rope", {"rotary_dim": m.rot_dims, "theta": m.rot_base, "style": "interleaved",
                                         "max_positions": DEFAULT_MAX_POSITIONS}) if m.rot_dims else None
            parts = {"norm1": norm,
                     "mixer": PartSpec("latent_attention", {
                         "hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim,
                         "value_dim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": cfg.eps,
                         "own_cache": m.kv_from is None, "position": position})}
            if layer.mlp is not None:
                f = layer.mlp
                parts["ffn"] = PartSpec("grouped_topk_moe", {
                    "hidden_size": cfg.width, "intermediate_size": f.ff, "num_experts": f.experts, "top": f.top,
                    "groups": f.groups, "keep_groups": f.keep, "router_scale": f.scale, "act": "silu"})
            layers.append(LayerSpec("parallel", parts, f"l{i}.", {"norm1": "norm1.", "mixer": "mix.", "ffn": "mlp."}))
            order.append(LayerCall(i, cache_of=m.kv_from))
            stored[f"l{i}.norm1.weight"] = f"l{i}.norm1"
        stored.update({"embed.weight": "embed", "final.norm.weight": "final.norm", "head.weight": "head"})
        additions = ()
        if cfg.pair_table is not None:
            t = cfg.pair_table
            additions = ((PartSpec("pair_hash", {"hidden_size": cfg.width, "buckets": t.buckets, "mul_prev": t.mul_prev,
                                                 "mul_cur": t.mul_cur, "tensor": "bigram"}), ""),)
        return ModelSpec(
            architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width,
            max_positions=DEFAULT_MAX_POSITIONS, layers=tuple(layers), order=tuple(order), final_norm=norm,
            embed_name="embed.", final_norm_name="final.norm.", head_name="head.", embed_scale=cfg.embed_scale,
            embed_additions=additions, stored_names=stored)
