"""The step function shared by the layer-list decoders of the generation path (Kelutar, Golavik, Gubulorn): one `step()` runs a
PACKED batch (llark_b200.state_cache) -- requests that start, go on by a portion of their prompt or decode one token are
the same kernels with other numbers -- and returns fp32 logits for the rows that are asked for. A model's engine
subclasses this and says how tokens become the residual stream (`_embed`), what its layers do to it (`_run_layers`) and
how wanted rows become logits (`_logits`); slot handling, the step descriptor, validation and the order of things are
here. The engine is host-side orchestration only, like LlamaEngine: every FLOP is a C-ABI call."""
import torch

F32 = torch.float32


class LayerListEngine:
    max_positions = None  # most tokens a request may hold (None: no bound)

    def _init_device(self, device, dtype):
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError("llark_b200 has no CPU path: the engine needs a CUDA device (B200)")
        if dtype not in (torch.bfloat16, torch.float32):
            raise TypeError("dtype must be torch.bfloat16 or torch.float32")
        self.device, self.act = dev, dtype
        return dev

    # hooks ------------------------------------------------------------------------------------------------------
    def new_cache(self, n_slots=4):
        raise NotImplementedError

    def _embed(self, ids, st):
        raise NotImplementedError

    def _run_layers(self, cache, x, st, residuals):
        """x fp32 [n_tok, width] through every layer; appends the stream after each layer run to `residuals` if given."""
        raise NotImplementedError

    def _logits(self, x, rows):
        raise NotImplementedError

    # one step ---------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, cache, slots, tokens, want=None, return_residuals=False):
        """slots: the requests of this step; tokens[b]: the next token ids of request slots[b] (they continue at the
        position where the request stopped); want[b]: indices into tokens[b] whose logits are asked for (None: the last
        one of each). Returns fp32 logits [n_wanted, vocab] in the order of the requests and of `want` (None when nothing
        is wanted). The caches advance by the step's tokens."""
        lens = [len(t) for t in tokens]
        st = cache.layout(slots, lens)
        if self.max_positions is not None:
            for s, n in zip(slots, lens):
                if cache.length[s] + n > self.max_positions:
                    raise ValueError("a request grows past max_positions")
        cache.reserve_positions(max(cache.length[s] + n for s, n in zip(slots, lens)))  # per-position stores grow first
        flat = [int(t) for ts in tokens for t in ts]
        if flat and (min(flat) < 0 or max(flat) >= self.cfg.vocab):
            raise ValueError("token id outside the vocabulary")
        ids = torch.tensor(flat, dtype=torch.int32).to(self.device, non_blocking=True)
        if want is None:
            want = [[n - 1] for n in lens]
        for b, w in enumerate(want):
            if any(k < 0 or k >= lens[b] for k in w):
                raise ValueError("a wanted place lies outside the request's tokens")
        rows = [st.cu_host[b] + int(k) for b, w in enumerate(want) for k in w]
        x = self._embed(ids, st)
        residuals = [] if return_residuals else None
        x = self._run_layers(cache, x, st, residuals)
        cache.advance(slots, lens)
        logits = None
        if rows:
            idx = torch.tensor(rows, dtype=torch.int32).to(self.device, non_blocking=True)
            logits = self._logits(x, idx)
        if return_residuals:
            return logits, residuals
        return logits
