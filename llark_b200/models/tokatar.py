"""Tokatar: a small decoder-only language model whose layers put a norm before AND after each sublayer and gate the
sublayer's result by its own input:

    h = norm_a(x);   y = sublayer(h) * sigmoid(W_rg h + b_rg);   x <- x + ls * norm_b(y)

with norm(z) = z / sqrt(mean(z^2) + eps) * g, g ONE number per norm, and `ls` a learned vector (layer scale). The mixer of
a layer is one of three kinds of attention -- grouped-query attention with rotary positions in halves, soft-capped scores
and a mask by blocks of positions ("attention"); the same with biased projections, an RMS norm over the whole q and k
projections, interleaved rotary pairs, values stored rotated by their own position and a 1 in every softmax denominator
("attention_2"); latent attention over everything before, one gate per head ("latent_attention") -- and the feed-forward is
down(relu(up h)^2). The embedding is scaled, the head is a matrix of its own. The reference has no such model; it is
served the way the other native decoders are: configuration and weights from a checkpoint folder (config.json +
model.safetensors), the CUDA engine (llark_b200.engine_tokatar), the slot cache (llark_b200.state_cache), `generate()`
through llark_b200.generate and batches through llark_b200.scheduler.

config.json keys: architecture ("Tokatar"), vocab, width, embedding.scale, norm.eps, layers[] with type, mixer {...},
mlp (null | {kind: "dense", ff}).
  attention, attention_2:  heads, kv_heads, dim, vdim, scale, softcap (optional), mask.size (optional: without it every
                           earlier position is seen), rot {base, dims, scaling {factor, low, high, original} (optional)};
                           tensors q, k, v, g, o (+ q.b, k.b, v.b, q.norm, k.norm for attention_2)
  latent_attention:        heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}; tensors q, dkv, dkv.norm, uk, uv, g, o
Other tensors: embed, head, final.norm, l<i>.norm1 / norm1b / norm2 / norm2b (one number each), l<i>.ls1 / ls2 [width],
l<i>.rg1 / rg2 [width, width] with .b, l<i>.mlp.up / down.
"""
from dataclasses import dataclass, field
from typing import List, Optional

from llark_b200.models.native import NativeCausalLM

ARCHITECTURE = "Tokatar"
# the configuration's layer types and feed-forward kinds -> entries of llark_b200.mixers.MIXERS / FEED_FORWARDS
MIXER_TYPES = {"attention": "rotary_attention", "attention_2": "rotary_attention_vrot",
               "latent_attention": "latent_attention_causal"}
FEED_FORWARD_KINDS = {"dense": "dense"}


@dataclass
class TokatarLayer:
    type: str
    mixer: dict
    mlp: Optional[dict] = None


@dataclass
class TokatarConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float = 1.0
    layers: List[TokatarLayer] = field(default_factory=list)
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d):
        from llark_b200.mixers import FEED_FORWARDS, MIXERS

        if d.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} configuration: architecture = {d.get('architecture')!r}")
        layers = []
        for i, e in enumerate(d["layers"]):
            if e["type"] not in MIXER_TYPES or MIXER_TYPES[e["type"]] not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {e['type']!r} (known: {sorted(MIXER_TYPES)})")
            mlp = e.get("mlp")
            if mlp is not None and (mlp.get("kind") not in FEED_FORWARD_KINDS
                                    or FEED_FORWARD_KINDS[mlp["kind"]] not in FEED_FORWARDS):
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r} (known: {sorted(FEED_FORWARD_KINDS)})")
            layers.append(TokatarLayer(type=e["type"], mixer=dict(e["mixer"]), mlp=dict(mlp) if mlp else None))
        if not layers:
            raise ValueError("a model needs at least one layer")
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)), layers=layers,
                   eos_token_id=d.get("eos_token_id"), pad_token_id=d.get("pad_token_id"))

    def to_dict(self):
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "embedding": {"scale": self.embedding_scale},
                "layers": [{"type": l.type, "mixer": l.mixer, "mlp": l.mlp} for l in self.layers]}


class TokatarForCausalLM(NativeCausalLM):
    """Inference-only model object: configuration + engine (llark_b200.models.native.NativeCausalLM)."""
    config_class = TokatarConfig

    @staticmethod
    def engine_class():
        from llark_b200.engine_tokatar import TokatarEngine

        return TokatarEngine
