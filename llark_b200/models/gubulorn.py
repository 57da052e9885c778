"""Gubulorn: a small decoder-only language model with the norm AFTER each residual sum, x <- norm(alpha x + sublayer(x)),
assembled from a per-layer list of mixers -- a gated delta rule with one decay per head ("delta"), or causal attention with
a sink and a state-space (Mamba-2) mixer side by side on the same input ("parallel") -- and feed-forwards that are either a
clamped gated unit or a routed mixture of experts (softmax router, choice with a stored correction, experts that hand their
input through). Embeddings are normed, the head is its own matrix, logits are scaled and soft-capped. The reference has no
such model; it is served the way the other native decoders are: configuration and weights from a checkpoint folder
(config.json + model.safetensors), the CUDA engine (llark_b200.engine_gubulorn), the slot cache (llark_b200.state_cache),
`generate()` through llark_b200.generate and batches through llark_b200.scheduler.

config.json keys: architecture ("Gubulorn"), vocab, width, norm.eps, postln_alpha, logit_scale, logit_softcap, layers[] with
type ("delta" | "parallel"), mixer {...}, mlp (null | {kind: "dense", ff, limit} | {kind: "moe", expert.ff, router {experts,
identity, top, groups {count, keep}}}).
  delta mixer:     heads, kv_heads, dim, vdim, conv;  tensors q, k, v (+ .conv each), b, a, A_log, dt_bias, g, norm, o
  parallel mixer:  left  {heads, kv_heads, dim, vdim, scale, q_temp {coef, every}};  tensors left.q, left.k, left.v,
                         left.q.norm, left.k.norm, left.sink, left.g, left.o, left.out
                   right {heads, vdim, state, groups, norm_groups, conv};  tensors right.in, right.conv, right.conv.b,
                         right.dt_bias, right.A_log, right.D, right.norm, right.o, right.out
Other tensors: embed, embed.norm, final.norm, head, l<i>.norm1, l<i>.norm2, l<i>.mlp.gate / up / down (dense),
l<i>.mlp.router, l<i>.mlp.correction, l<i>.mlp.e<j>.gate / up / down (moe). Norm weights are stored around zero (the norm
multiplies by 1 + w) except the plain ones inside the mixers.
"""
from dataclasses import dataclass, field
from typing import List, Optional

from llark_b200.models.native import NativeCausalLM

ARCHITECTURE = "Gubulorn"
LAYER_TYPES = ("delta", "parallel")
# the configuration's feed-forward kinds -> entries of llark_b200.mixers.FEED_FORWARDS
FEED_FORWARD_KINDS = {"dense": "clamped_glu", "moe": "moe_softmax_bias"}


@dataclass
class GubulornLayer:
    type: str
    mixer: dict
    mlp: Optional[dict] = None


@dataclass
class GubulornConfig:
    vocab: int
    width: int
    eps: float
    alpha: float
    logit_scale: float = 1.0
    logit_softcap: Optional[float] = None
    layers: List[GubulornLayer] = field(default_factory=list)
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d):
        from llark_b200.mixers import MIXERS

        if d.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} configuration: architecture = {d.get('architecture')!r}")
        layers = []
        for i, e in enumerate(d["layers"]):
            if e["type"] not in LAYER_TYPES or e["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {e['type']!r} (known: {list(LAYER_TYPES)})")
            mlp = e.get("mlp")
            if mlp is not None and mlp.get("kind") not in FEED_FORWARD_KINDS:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r} (known: {sorted(FEED_FORWARD_KINDS)})")
            layers.append(GubulornLayer(type=e["type"], mixer=dict(e["mixer"]), mlp=dict(mlp) if mlp else None))
        cap = d.get("logit_softcap")
        if cap is not None and not float(cap) > 0.0:
            raise ValueError("logit_softcap must be positive (or absent)")
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]),
                   alpha=float(d.get("postln_alpha", 1.0)), logit_scale=float(d.get("logit_scale", 1.0)),
                   logit_softcap=float(cap) if cap is not None else None, layers=layers,
                   eos_token_id=d.get("eos_token_id"), pad_token_id=d.get("pad_token_id"))

    def to_dict(self):
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "postln_alpha": self.alpha, "logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap,
                "layers": [{"type": l.type, "mixer": l.mixer, "mlp": l.mlp} for l in self.layers]}


class GubulornForCausalLM(NativeCausalLM):
    """Inference-only model object: configuration + engine (llark_b200.models.native.NativeCausalLM)."""
    config_class = GubulornConfig

    @staticmethod
    def engine_class():
        from llark_b200.engine_gubulorn import GubulornEngine

        return GubulornEngine
