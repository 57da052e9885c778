"""Execution schedule of the Tokatar decoder on the generation path: a list of layers, each sublayer between two norms and
gated by its own input,

    h = norm1(x);   x = x + ls1 * norm1b(mixer(h) * sigmoid(rg1 h + b1))
    h = norm2(x);   x = x + ls2 * norm2b(ff(h)    * sigmoid(rg2 h + b2))        only in layers that have a feed-forward

with norm(z) = z / sqrt(mean(z^2) + eps) * g (g one number) and ls a vector. The mixer is chosen per layer from
llark_b200.mixers.MIXERS through llark_b200.models.tokatar.MIXER_TYPES (three kinds of attention), the feed-forward from
FEED_FORWARDS. Logits are head(final_norm(x)).

Gate, norm of the result, layer scale, residual sum AND the next sublayer's input norm are ONE kernel
(llark_seq_gated_norm_add): the stream is read and written once per sublayer. The mixer's gate projection rg1 reads the
same input as q / k / v / g and is part of the mixer's fused input GEMM (`side`). The step function is
llark_b200.engine_seq.LayerListEngine.step; keys and values live in a llark_b200.state_cache.StateCache (rings of
mask.size entries for the masked attentions, per-position stores that grow for the latent attention). Precision: the
residual stream, norms, rotation angles, attention scores and softmax are fp32 in both modes, and every projection that
feeds one of them is written in fp32 by its GEMM; matrix products and the activations between them are bf16 with fp32
accumulation (dtype=torch.bfloat16) or true fp32 (dtype=torch.float32).
"""
import torch

from . import ops
from .engine_seq import LayerListEngine
from .mixers import FEED_FORWARDS, MIXERS, _pad_rows
from .models.tokatar import FEED_FORWARD_KINDS, MIXER_TYPES
from .state_cache import StateCache

F32 = torch.float32


class TokatarEngine(LayerListEngine):
    def __init__(self, config, weights, device, dtype=torch.bfloat16):
        """config: llark_b200.models.tokatar.TokatarConfig; weights: name -> tensor (any device / float dtype)."""
        dev = self._init_device(device, dtype)
        self.cfg = config
        C = config.width

        def scalar(name):  # a norm's one number, as a vector for the row kernels
            v = weights[name].to(device=dev, dtype=F32)
            if v.numel() != 1:
                raise ValueError(f"{name} must be one number")
            return v.reshape(1).expand(C).contiguous()

        def vector(name):
            v = weights[name].to(device=dev, dtype=F32).contiguous()
            if tuple(v.shape) != (C,):
                raise ValueError(f"{name} does not fit the width")
            return v

        self.embed = weights["embed"].to(device=dev, dtype=dtype).contiguous()
        head = weights["head"].to(device=dev, dtype=dtype)
        if tuple(self.embed.shape) != (config.vocab, C) or tuple(head.shape) != (config.vocab, C):
            raise ValueError("embed / head do not fit vocab x width")
        self.head = _pad_rows(head)  # logits of the padding rows are cut off
        self.final_norm = scalar("final.norm")
        self._packed = []
        for i, layer in enumerate(config.layers):
            p = f"l{i}."
            mixer_cls = MIXERS[MIXER_TYPES[layer.type]]
            pk = {"mixer": mixer_cls.Weights(weights, p + "mix.", layer.mixer, C, dev, dtype, side=(p + "rg1", p + "rg1.b")),
                  "norm1": scalar(p + "norm1"), "post1": (scalar(p + "norm1b") * vector(p + "ls1")).contiguous(),
                  "ff": None}
            if pk["mixer"].side_n != C:
                raise ValueError(f"{p}rg1 does not fit width x width")
            if layer.mlp is not None:
                pk["ff_kind"] = FEED_FORWARD_KINDS[layer.mlp["kind"]]
                pk["ff"] = FEED_FORWARDS[pk["ff_kind"]].Weights(weights, p + "mlp.", layer.mlp, C, dev, dtype)
                pk["norm2"] = scalar(p + "norm2")
                pk["post2"] = (scalar(p + "norm2b") * vector(p + "ls2")).contiguous()
                pk["rg2"] = weights[p + "rg2"].to(device=dev, dtype=dtype).contiguous()
                pk["rg2_b"] = vector(p + "rg2.b")
                if tuple(pk["rg2"].shape) != (C, C):
                    raise ValueError(f"{p}rg2 does not fit width x width")
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
                           "mixer": MIXERS[MIXER_TYPES[layer.type]](pk["mixer"], cache, cfg.eps, self.act, self.max_positions),
                           "ff": FEED_FORWARDS[pk["ff_kind"]](pk["ff"], self.act) if pk["ff"] is not None else None})
        cache.layers = layers
        return cache

    # ------------------------------------------------------------------------------------------ one step (hooks)
    def _embed(self, ids, st):
        return ops.seq_embed(ids, st, self.embed, None, self.cfg.embedding_scale)

    def _run_layers(self, cache, x, st, residuals):
        eps = self.cfg.eps
        entries = cache.layers
        # the first input norm (one part over the width); every later one rides on a residual kernel
        h = ops.seq_group_rmsnorm(x, entries[0]["pk"]["norm1"], 1, eps, out_dtype=self.act)
        for i, entry in enumerate(entries):
            pk = entry["pk"]
            nxt = entries[i + 1]["pk"]["norm1"] if i + 1 < len(entries) else None
            mixer = entry["mixer"]
            y = mixer.forward(h, st, cache)
            if entry["ff"] is None:
                x, h = self._residual(x, y, pk["post1"], mixer.side, nxt)
            else:
                x, h = self._residual(x, y, pk["post1"], mixer.side, pk["norm2"])
                gate = ops.linear(h, pk["rg2"], bias=pk["rg2_b"], out_dtype=F32)
                x, h = self._residual(x, entry["ff"].forward(h), pk["post2"], gate, nxt)
            if residuals is not None:
                residuals.append(x)
        return x

    def _residual(self, x, y, w_post, gate, w_next):
        if w_next is None:
            return ops.seq_gated_norm_add(x, y, w_post, self.cfg.eps, gate=gate), None
        return ops.seq_gated_norm_add(x, y, w_post, self.cfg.eps, gate=gate, w_next=w_next, act=self.act)

    def _logits(self, x, rows):
        hn = ops.seq_group_rmsnorm(x, self.final_norm, 1, self.cfg.eps, out_dtype=self.act, rows=rows)
        return ops.linear(hn, self.head, out_dtype=F32)[:, :self.cfg.vocab]
