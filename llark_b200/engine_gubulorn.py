"""Execution schedule of the Gubulorn decoder on the generation path: a list of layers with the norm after each sum,

    x  = norm1(alpha * x + mixer(x))
    x  = norm2(alpha * x + ff(x))               only in layers that have a feed-forward

with norm(s) = s / sqrt(mean(s^2) + eps) * (1 + w), the sublayers reading x itself. The mixer is chosen per layer from
llark_b200.mixers.MIXERS ("delta": gated delta rule with a decay per head; "parallel": attention with a sink beside a
state-space mixer, whose RMS-normed outputs are averaged), the feed-forward from FEED_FORWARDS (a clamped gated unit, or a
mixture of experts with a softmax router). The token embedding is normed before the first layer; the logits are
head(norm(x)) * logit_scale, soft-capped by tanh.

Each sum and its norm are ONE kernel (llark_seq_post_norm): it also norms and averages the two outputs of a parallel mixer
and takes the weighted sum over a token's chosen experts, so neither is ever written out. The step function is
llark_b200.engine_seq.LayerListEngine.step; state lives in a llark_b200.state_cache.StateCache (recurrent states and
convolution carries per slot, keys and values per position in stores that grow). Precision: the residual stream, norms,
attention scores and softmax, router, decays, step sizes, gates of the recurrences and their states are fp32 in both modes;
matrix products and the activations between them are bf16 with fp32 accumulation (dtype=torch.bfloat16) or true fp32
(dtype=torch.float32).
"""
import torch

from . import ops
from .engine_seq import LayerListEngine
from .mixers import FEED_FORWARDS, MIXERS, _pad_rows
from .models.gubulorn import FEED_FORWARD_KINDS
from .state_cache import StateCache

F32 = torch.float32


class GubulornEngine(LayerListEngine):
    def __init__(self, config, weights, device, dtype=torch.bfloat16):
        """config: llark_b200.models.gubulorn.GubulornConfig; weights: name -> tensor (any device / float dtype)."""
        dev = self._init_device(device, dtype)
        self.cfg = config
        C = config.width

        def one_plus(name):
            v = weights[name].to(device=dev, dtype=F32)
            if tuple(v.shape) != (C,):
                raise ValueError(f"{name} does not fit the width")
            return (1.0 + v).contiguous()

        self.embed = weights["embed"].to(device=dev, dtype=dtype).contiguous()
        head = weights["head"].to(device=dev, dtype=dtype)
        if tuple(self.embed.shape) != (config.vocab, C) or tuple(head.shape) != (config.vocab, C):
            raise ValueError("embed / head do not fit vocab x width")
        self.head = _pad_rows(head)  # logits of the padding rows are cut off
        self.embed_norm, self.final_norm = one_plus("embed.norm"), one_plus("final.norm")
        self._packed = []
        for i, layer in enumerate(config.layers):
            p = f"l{i}."
            pk = {"mixer": MIXERS[layer.type].Weights(weights, p + "mix.", layer.mixer, C, dev, dtype),
                  "norm1": one_plus(p + "norm1"), "ff": None, "ff_kind": None, "norm2": None}
            if layer.mlp is not None:
                pk["ff_kind"] = FEED_FORWARD_KINDS[layer.mlp["kind"]]
                pk["ff"] = FEED_FORWARDS[pk["ff_kind"]].Weights(weights, p + "mlp.", layer.mlp, C, dev, dtype)
            if layer.mlp is not None or p + "norm2" in weights:
                pk["norm2"] = one_plus(p + "norm2")
            self._packed.append(pk)

    # ------------------------------------------------------------------------------------------ state
    def new_cache(self, n_slots=4):
        """A StateCache with every layer's stores declared. The per-position stores start with room for max_positions
        tokens per request when that is set, and grow otherwise."""
        cfg = self.cfg
        cache = StateCache(self.device, n_slots=n_slots, positions=self.max_positions or 256)
        layers = []
        for pk, layer in zip(self._packed, cfg.layers):
            layers.append({"pk": pk,
                           "mixer": MIXERS[layer.type](pk["mixer"], cache, cfg.eps, self.act, self.max_positions),
                           "ff": FEED_FORWARDS[pk["ff_kind"]](pk["ff"], self.act) if pk["ff"] is not None else None})
        cache.layers = layers
        return cache

    # ------------------------------------------------------------------------------------------ one step (hooks)
    def _embed(self, ids, st):
        return ops.seq_embed(ids, st, self.embed, None, 1.0)

    def _run_layers(self, cache, x, st, residuals):
        cfg = self.cfg
        x, xa = ops.seq_post_norm(x, 1.0, self.embed_norm, cfg.eps, act=self.act)  # the embedding's own norm
        for entry in cache.layers:
            pk = entry["pk"]
            outs, scale = entry["mixer"].branches(xa, st, cache)
            (y1, w1), (y2, w2) = outs[0], (outs[1] if len(outs) > 1 else (None, None))
            x, xa = ops.seq_post_norm(x, cfg.alpha, pk["norm1"], cfg.eps, y1=y1, w1=w1, y2=y2, w2=w2, branch_scale=scale,
                                      act=self.act)
            if entry["ff"] is not None:
                x, xa = entry["ff"].post_norm(x, xa, cfg.alpha, pk["norm2"], cfg.eps, self.act)
            elif pk["norm2"] is not None:
                x, xa = ops.seq_post_norm(x, cfg.alpha, pk["norm2"], cfg.eps, act=self.act)
            if residuals is not None:
                residuals.append(x)
        return x

    def _logits(self, x, rows):
        hn = ops.seq_rmsnorm_rows(x, rows, self.final_norm, self.cfg.eps, self.act)
        z = ops.linear(hn, self.head, out_dtype=F32)
        ops.seq_logit_cap_(z, self.cfg.logit_scale, self.cfg.logit_softcap)
        return z[:, :self.cfg.vocab]
