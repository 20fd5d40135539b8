"""Gepadra as a ``ModelSpec``.

Every layer is a parallel block with a norm of its own for each branch, x <- x + (mixer(n1(x)) + ff(n2(x))); the
norms are RMS norms whose stored scale is an offset from one.  The mixer is either grouped-query attention with
biases, a partial rotation of the leading head dims, a sliding window that keeps a sequence's first tokens, a
learned sink logit per head in the softmax and values blended with those of the first such layer
(``attention``), or an mLSTM matrix memory with capped exponential gates (``mlstm``), whose state is a slab of
the cache manager.  The feed-forward is a clamped gated unit (``gated_mlp`` with ``act: swish_clamped``) or a
mixture of small ungated experts with a sigmoid router whose scores scale the experts' inputs, beside a shared
expert behind a sigmoid gate (``sigmoid_topk_moe``).  The output head is the embedding table.  Checkpoints name
tensors ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*`` and ``final.norm``.
The reference registers its families in one table keyed by the checkpoint's architecture string
(crates/thuban_architectures/src/loader.rs:39-60).
"""
from __future__ import annotations

from ..config.gepadra import DEFAULT_MAX_POSITIONS, GepadraConfig
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..registry import ARCHITECTURES

SWISH_SLOPE = 1.702       # the design fixes the slope of the gated unit's sigmoid


@ARCHITECTURES.register("Gepadra")
class GepadraArchitecture:
    config_class = GepadraConfig

    @staticmethod
    def parse_config(d: dict) -> GepadraConfig:
        return GepadraConfig.from_dict(d)

    @staticmethod
    def model_spec(cfg: GepadraConfig) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.eps, "weight_offset": 1.0})
        layers, order, stored = [], [], {}
        first_mix = None          # the first layer that blends values: the others read its values
        for i, layer in enumerate(cfg.layers):
            m, pre = layer.mixer, f"l{i}."
            if layer.type == "attention":
                position = PartSpec("rope", {"rotary_dim": m.rot_dims, "theta": m.rot_base, "style": "half",
                                             "max_positions": DEFAULT_MAX_POSITIONS}) if m.rot_dims else None
                role = None
                if m.v_mix:
                    role = "source" if first_mix is None else "blend"
                    first_mix = i if first_mix is None else first_mix
                params = {"hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                          "value_dim": m.vdim, "window": m.window, "keep_first": m.keep_first, "qkv_bias": True,
                          "scale": m.scale, "sinks": True, "position": position}
                if role is not None:
                    params["value_mix"] = role      # such a layer stores a blend weight, also the first, which ignores it
                mixer = PartSpec("attention", params)
                for ours, theirs in (("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"),
                                     ("o_proj.weight", "o"), ("q_proj.bias", "q.b"), ("k_proj.bias", "k.b"),
                                     ("v_proj.bias", "v.b"), ("sinks", "sink"), ("value_mix", "vmix")):
                    stored[f"{pre}mix.{ours}"] = f"{pre}mix.{theirs}"
            else:
                mixer = PartSpec("mlstm", {"hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim,
                                           "value_dim": m.vdim, "gate_cap": m.gate_cap, "norm_eps": cfg.eps})
            parts = {"norm1": norm, "mixer": mixer}
            names = {"norm1": "norm1.", "mixer": "mix.", "norm2": "norm2.", "ffn": "mlp."}
            stored[f"{pre}norm1.weight"] = f"{pre}norm1"
            f = layer.mlp
            if f is not None:
                parts["norm2"] = norm
                stored[f"{pre}norm2.weight"] = f"{pre}norm2"
                if hasattr(f, "limit"):
                    parts["ffn"] = PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": f.ff,
                                                          "act": "swish_clamped", "act_slope": SWISH_SLOPE,
                                                          "act_limit": f.limit})
                    for ours, theirs in (("gate_proj.weight", "gate"), ("up_proj.weight", "up"), ("down_proj.weight", "down")):
                        stored[f"{pre}mlp.{ours}"] = f"{pre}mlp.{theirs}"
                else:
                    parts["ffn"] = PartSpec("sigmoid_topk_moe", {
                        "hidden_size": cfg.width, "intermediate_size": f.ff, "num_experts": f.experts, "top": f.top,
                        "shared_intermediate_size": f.shared_ff, "act": "gelu"})
            layers.append(LayerSpec("parallel_two_norms", parts, pre, names))
            order.append(LayerCall(i))
        stored.update({"embed.weight": "embed", "final.norm.weight": "final.norm"})
        return ModelSpec(
            architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width,
            max_positions=DEFAULT_MAX_POSITIONS, layers=tuple(layers), order=tuple(order), final_norm=norm,
            embed_name="embed.", final_norm_name="final.norm.", tie_word_embeddings=True, stored_names=stored)
