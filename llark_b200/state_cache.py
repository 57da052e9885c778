"""Per-request memory of the generation path: a slot allocator over device stores, and the packed-step descriptor.

The Llama path's KVCache (engine.py) holds one prompt batch of equal lengths. Decoders whose layers keep other things
than a growing key / value list (a ring of the last `window` keys, a recurrent state, the last inputs of a short
convolution) and whose requests come and go with different lengths use this instead: every layer registers the stores
it needs (`add_store`), a request owns one SLOT = one row of every store from `alloc()` to `release()`, and the kernels
index the stores by slot. Stores of equal shape are stacked into one tensor [n_layers_of_that_kind, n_slots, ...], so
starting a request zeroes each kind with one fill and a layer's view [n_slots, ...] stays contiguous. Stores grow by
doubling when the slots run out. A store that holds one entry per POSITION of a request (the keys and values of an
attention that looks back without a bound) is declared with per_position=True: its first axis is `positions` entries
long for every such store of the cache and doubles (`reserve_positions`) before a step that would outgrow it, old entries
kept in place.

Sized for one B200: a ring is min(window, max_positions) entries per slot whatever the sequence length; a recurrent
state is heads x dim x vdim fp32 per slot.
"""
import torch


class StepLayout:
    """One packed step on the device: request b brings lens[b] tokens that start at position pos0[b] of its sequence and
    owns slot slots[b]. tok_seq[t] = request of row t; cu[b] = first row of request b. One pinned host buffer, one copy."""

    def __init__(self, lens, pos0, slots, device):
        n_seq = len(lens)
        n_tok = int(sum(lens))
        if n_seq == 0 or min(lens) <= 0:
            raise ValueError("a step needs at least one token for every request in it")
        host = torch.empty(n_tok + 4 * n_seq + 1, dtype=torch.int32, pin_memory=torch.device(device).type == "cuda")
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + int(n))
        seq = []
        for b, n in enumerate(lens):
            seq.extend([b] * int(n))
        host[:n_tok] = torch.tensor(seq, dtype=torch.int32)
        host[n_tok:n_tok + n_seq + 1] = torch.tensor(cu, dtype=torch.int32)
        host[n_tok + n_seq + 1:n_tok + 2 * n_seq + 1] = torch.tensor([int(p) for p in pos0], dtype=torch.int32)
        host[n_tok + 2 * n_seq + 1:n_tok + 3 * n_seq + 1] = torch.tensor([int(s) for s in slots], dtype=torch.int32)
        host[n_tok + 3 * n_seq + 1:] = torch.tensor([int(n) for n in lens], dtype=torch.int32)
        dev = host.to(device, non_blocking=True)
        self._host = host  # keeps the pinned buffer alive until the copy has run
        self.tok_seq = dev[:n_tok]
        self.cu = dev[n_tok:n_tok + n_seq + 1]
        self.pos0 = dev[n_tok + n_seq + 1:n_tok + 2 * n_seq + 1]
        self.slot = dev[n_tok + 2 * n_seq + 1:n_tok + 3 * n_seq + 1]
        self.lens_dev = dev[n_tok + 3 * n_seq + 1:]
        self.device, self.slots_host, self._chunks = device, [int(s) for s in slots], {}
        self.n_tok, self.n_seq = n_tok, n_seq
        self.max_len = int(max(lens))
        self.lens, self.cu_host, self.pos0_host = [int(n) for n in lens], cu, [int(p) for p in pos0]


class _Chunks:
    pass


def _step_chunks(self, length):
    """The step cut into work items of at most `length` consecutive rows of one request (for scans that run long
    prompts as independent chunks): row0 / n per item, index = 0 .. n_items-1, minus1 = -1 everywhere, last_slot = the
    request's slot on its last item and -1 elsewhere, seq_item0[b] = first item of request b. Built once per step."""
    if length in self._chunks:
        return self._chunks[length]
    row0, n, last, seq0 = [], [], [], [0]
    for b, ln in enumerate(self.lens):
        for lo in range(0, ln, length):
            row0.append(self.cu_host[b] + lo)
            n.append(min(length, ln - lo))
            last.append(self.slots_host[b] if lo + length >= ln else -1)
        seq0.append(len(row0))
    k = len(row0)
    host = torch.tensor(row0 + n + list(range(k)) + [-1] * k + last + seq0, dtype=torch.int32)
    if torch.device(self.device).type == "cuda":
        host = host.pin_memory()
    dev = host.to(self.device, non_blocking=True)
    c = _Chunks()
    c._host = host
    c.n_items = k
    c.row0, c.n, c.index, c.minus1, c.last_slot = (dev[i * k:(i + 1) * k] for i in range(5))
    c.seq_item0 = dev[5 * k:]
    self._chunks[length] = c
    return c


StepLayout.chunks = _step_chunks


class StateCache:
    def __init__(self, device, n_slots=4, positions=256):
        self.device = torch.device(device)
        self.n_slots = int(n_slots)
        self.positions = max(int(positions), 1)  # entries per slot of the per-position stores
        self.has_per_position = False
        self._decl = []      # (shape, dtype, zero_on_alloc) per handle
        self._groups = {}    # (shape, dtype, zero) -> [handles]
        self._tensors = {}   # group key -> stacked tensor [count, n_slots, *shape]
        self._where = {}     # handle -> (group key, index in group)
        self._free = list(range(self.n_slots - 1, -1, -1))
        self.length = {}     # slot -> tokens the request holds so far
        self.allocs = 0      # how often a slot was handed out (a reused slot counts again)

    # ------------------------------------------------------------------------------------------ stores
    def add_store(self, shape, dtype, zero_on_alloc, per_position=False):
        """Declare a per-slot store of `shape`; returns a handle for view(). All stores must be declared before the
        first alloc(). per_position: the store is [positions, *shape] per slot and grows with reserve_positions()."""
        if self._tensors:
            raise RuntimeError("stores must be declared before the cache is used")
        key = (tuple(int(s) for s in shape), dtype, bool(zero_on_alloc), bool(per_position))
        self.has_per_position = self.has_per_position or bool(per_position)
        h = len(self._decl)
        self._decl.append(key)
        self._groups.setdefault(key, []).append(h)
        self._where[h] = (key, len(self._groups[key]) - 1)
        return h

    def _build(self):
        for key, handles in self._groups.items():
            shape, dtype, _, per_pos = key
            lead = (self.positions,) if per_pos else ()
            self._tensors[key] = torch.zeros((len(handles), self.n_slots) + lead + shape, device=self.device, dtype=dtype)

    def view(self, handle):
        """The store as [n_slots, *shape] (contiguous). Fetch it every step: growing the cache replaces the tensors."""
        if not self._tensors:
            self._build()
        key, i = self._where[handle]
        return self._tensors[key][i]

    def bytes_per_slot(self):
        n = 0
        for key, handles in self._groups.items():
            shape, dtype, _, per_pos = key
            e = self.positions if per_pos else 1
            for s in shape:
                e *= s
            n += e * len(handles) * torch.empty((), dtype=dtype).element_size()
        return n

    # ------------------------------------------------------------------------------------------ slots
    def _grow(self):
        old = self.n_slots
        self.n_slots = old * 2
        for key, t in list(self._tensors.items()):
            bigger = torch.zeros((t.shape[0], self.n_slots) + t.shape[2:], device=self.device, dtype=t.dtype)
            bigger[:, :old].copy_(t)
            self._tensors[key] = bigger
        self._free.extend(range(self.n_slots - 1, old - 1, -1))

    def reserve_positions(self, n):
        """Make room for requests of up to n tokens in the per-position stores (doubling; entries keep their place)."""
        if n <= self.positions or not self.has_per_position:
            return
        new = self.positions
        while new < n:
            new *= 2
        if self._tensors:
            for key, t in list(self._tensors.items()):
                if key[3]:
                    bigger = torch.zeros(t.shape[:2] + (new,) + t.shape[3:], device=self.device, dtype=t.dtype)
                    bigger[:, :, :self.positions].copy_(t)
                    self._tensors[key] = bigger
        self.positions = new

    def alloc(self):
        """A slot for a new request: its recurrent / convolution state starts at zero, it holds no tokens."""
        if not self._tensors:
            self._build()
        if not self._free:
            self._grow()
        slot = self._free.pop()
        for key, t in self._tensors.items():
            if key[2]:
                t[:, slot].zero_()
        self.length[slot] = 0
        self.allocs += 1
        return slot

    def release(self, slot):
        if slot not in self.length:
            raise KeyError(f"slot {slot} is not in use")
        del self.length[slot]
        self._free.append(slot)

    def in_use(self):
        return sorted(self.length)

    def tokens_held(self):
        return sum(self.length.values())

    def layout(self, slots, lens):
        """StepLayout for requests `slots` bringing `lens` new tokens each; positions continue where each stopped."""
        for s in slots:
            if s not in self.length:
                raise KeyError(f"slot {s} is not in use")
        if len(set(slots)) != len(slots):
            raise ValueError("a request can appear once in a step")
        return StepLayout(lens, [self.length[s] for s in slots], slots, self.device)

    def advance(self, slots, lens):
        for s, n in zip(slots, lens):
            self.length[s] += int(n)
