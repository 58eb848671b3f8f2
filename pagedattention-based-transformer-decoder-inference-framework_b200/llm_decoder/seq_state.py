"""SequenceStateCache -- what a live request holds on the device between two steps, next to its K/V pages:

  * a STATE SLOT: one row in every per-layer float state tensor (the previous token's normalised row for token
    shift, a recurrent layer's hidden state, ...).  Slots come from a free list and are zeroed when handed out, so a
    new sequence starts from the all-zero state whatever the slot held before;
  * its tiles in the paged K/V pools of the attention layers (one KVTileCache per layer, table row = slot), registered
    as its tokens arrive and released when it ends.

The pools are sized for `max_tokens` live tokens (each request rounded up to whole tiles), not for the sum of all
requests: pages and slots are used again, and running out is an error, never an eviction of a live request."""
import numpy as np
import torch

from .host_stage import to_device as _to_device
from .kv_tile_cache import KVTileCache


class RaggedBatch:
    """Device-side description of one step's rows (see csrc/seq_ops.cu): per row (slot, position, previous row or -1),
    per portion (first row, length, slot).  Built by SequenceStateCache.make_batch."""

    def __init__(self, ids, row_slot, row_pos, row_prev, seq_start, seq_len, seq_slot, portions, device):
        i32 = dict(dtype=torch.int32)
        host = torch.from_numpy(np.stack([np.asarray(a, dtype=np.int32) for a in (ids, row_slot, row_pos, row_prev)]))
        self.rows = len(ids)
        self.num_seqs = len(seq_start)
        self.portions = portions                      # host list of (first row, length, slot, first position)
        dev_rows = _to_device(host, device)
        self.ids, self.row_slot, self.row_pos, self.row_prev = dev_rows[0], dev_rows[1], dev_rows[2], dev_rows[3]
        seqs = torch.tensor([seq_start, seq_len, seq_slot], **i32)
        dev_seqs = _to_device(seqs, device)
        self.seq_start, self.seq_len, self.seq_slot = dev_seqs[0], dev_seqs[1], dev_seqs[2]
        self.device = device
        self._cache = {}

    def query_tiles(self, tile_tokens, big_tokens=0, big_from=0):
        """The work lists of the attention kernels: every portion cut into runs of consecutive tokens, as [n, 4] int32
        device tensors (first row, tokens, slot, first position).  Three lists, keyed by the kernel's tile kind:
        1 = portions of ONE token (decoded tokens: the streaming kernel), 2 = portions of at least `big_from` tokens in
        runs of `big_tokens` (the tensor-core kernel; none when big_tokens is 0), 0 = the rest in runs of `tile_tokens`.
        Each comes as (tensor, count, longest context) or None."""
        key = ("qt", tile_tokens, big_tokens, big_from)
        if key not in self._cache:
            groups = {0: [], 1: [], 2: []}
            for r0, n, slot, p0 in self.portions:
                kind = 1 if n == 1 else 2 if big_tokens and n >= big_from else 0
                step = big_tokens if kind == 2 else tile_tokens
                for o in range(0, n, step):
                    groups[kind].append((r0 + o, min(step, n - o), slot, p0 + o))
            out = {}
            for kind, tiles in groups.items():
                if not tiles:
                    out[kind] = None
                    continue
                t = torch.tensor(tiles, dtype=torch.int32).reshape(-1, 4)
                out[kind] = (_to_device(t, self.device), len(tiles), max(p + m for _r, m, _s, p in tiles))
            self._cache[key] = out
        return self._cache[key]

    def chunk_items(self, chunk):
        """Every portion cut into runs of at most `chunk` consecutive tokens (0: whole portions), in portion order, as work
        items of the convolution and matrix-state scan kernels: ([n, 4] int32 device tensor of (first row, tokens, slot,
        offset of the first token within its portion), n, first item per portion, items per portion)."""
        key = ("ci", chunk)
        if key not in self._cache:
            items, s0, sn = [], [], []
            for r0, n, slot, _p0 in self.portions:
                s0.append(len(items))
                step = chunk if chunk > 0 else n
                for o in range(0, n, step):
                    items.append((r0 + o, min(step, n - o), slot, o))
                sn.append(len(items) - s0[-1])
            t = torch.tensor(items, dtype=torch.int32).reshape(-1, 4)
            b = torch.tensor([s0, sn], dtype=torch.int32)
            t, b = _to_device(t, self.device), _to_device(b, self.device)
            self._cache[key] = (t, len(items), b[0], b[1])
        return self._cache[key]

    def scan_chunks(self, chunk):
        """Chunk lists of the chunked recurrent scan: (chunk_start, chunk_len, seq_chunk0, seq_nchunks) device int32
        tensors and the chunk count."""
        key = ("sc", chunk)
        if key not in self._cache:
            cs, cl, s0, sn = [], [], [], []
            for r0, n, _slot, _p0 in self.portions:
                s0.append(len(cs))
                for o in range(0, n, chunk):
                    cs.append(r0 + o)
                    cl.append(min(chunk, n - o))
                sn.append(len(cs) - s0[-1])
            a = torch.tensor([cs, cl], dtype=torch.int32)
            b = torch.tensor([s0, sn], dtype=torch.int32)
            a, b = _to_device(a, self.device), _to_device(b, self.device)
            self._cache[key] = (a[0], a[1], b[0], b[1], len(cs))
        return self._cache[key]


class SequenceStateCache:
    def __init__(self, max_seqs, max_tokens, tile_size=16, device=None):
        if max_seqs <= 0 or max_tokens <= 0 or tile_size <= 0:
            raise ValueError("SequenceStateCache: sizes must be positive")
        self.max_seqs, self.tile_size = int(max_seqs), int(tile_size)
        self.max_tiles = (int(max_tokens) + tile_size - 1) // tile_size      # tiles of the whole pool, per kv head
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._free_slots = list(range(self.max_seqs - 1, -1, -1))
        self._states = []           # float [max_seqs, width] tensors
        self._kv = []               # KVTileCache per attention layer
        self._len = {}              # slot -> tokens held

    # ---- set-up (by the model, once) --------------------------------------------------------------------------------
    def add_state(self, width):
        t = torch.zeros((self.max_seqs, int(width)), dtype=torch.float32, device=self.device)
        self._states.append(t)
        return t

    def add_kv_layer(self, kv_heads, key_dim, value_dim, dtype):
        """A paged pool for one attention layer: max_tiles * kv_heads pages; the table has one row per slot and lets a
        single request grow to the whole pool."""
        kvc = KVTileCache(dtype, device=self.device)
        kvc.init(self.max_tiles * int(kv_heads), self.tile_size, int(key_dim), int(value_dim))
        kvc.configure_table(self.max_seqs, int(kv_heads), self.max_tiles)
        kvc.evict_on_exhaustion = False
        self._kv.append(kvc)
        return kvc

    # ---- per request ------------------------------------------------------------------------------------------------
    def alloc(self):
        if not self._free_slots:
            raise RuntimeError("SequenceStateCache: no free state slot")
        slot = self._free_slots.pop()
        for t in self._states:
            t[slot].zero_()
        self._len[slot] = 0
        return slot

    def length(self, slot):
        return self._len[slot]

    def free_slots(self):
        return len(self._free_slots)

    def free_tokens(self):
        """Tokens that can still be taken (whole free tiles)."""
        if not self._kv:
            return 1 << 60
        return min(k.free_pages() // k.page_table_.num_heads_ for k in self._kv) * self.tile_size

    def extend(self, slot, n_new):
        """Reserve room for the next n_new tokens of `slot`: registers the tiles they touch in every attention layer's
        pool.  Returns the position of the first of them."""
        pos0 = self._len[slot]
        t0 = (pos0 + self.tile_size - 1) // self.tile_size
        t1 = (pos0 + n_new + self.tile_size - 1) // self.tile_size
        if t1 > self.max_tiles:
            raise RuntimeError("SequenceStateCache: request exceeds the pool")
        for kvc in self._kv:
            kvc.register_range(slot, t0, t1)
        self._len[slot] = pos0 + n_new
        return pos0

    def free(self, slot):
        for kvc in self._kv:
            kvc.release_beam(slot)
        del self._len[slot]
        self._free_slots.append(slot)

    # ---- batch description ------------------------------------------------------------------------------------------
    def make_batch(self, entries):
        """entries: [(slot, token ids)] in batch order, each slot at most once.  Extends every slot by its tokens and
        returns the RaggedBatch."""
        ids, row_slot, row_pos, row_prev = [], [], [], []          # one int32 array per portion
        seq_start, seq_len, seq_slot, portions = [], [], [], []
        seen = set()
        r0 = 0
        for slot, toks in entries:
            if slot in seen:
                raise ValueError("a sequence may appear once per step")
            seen.add(slot)
            n = len(toks)
            if n == 0:
                continue
            p0 = self.extend(slot, n)
            seq_start.append(r0)
            seq_len.append(n)
            seq_slot.append(slot)
            portions.append((r0, n, slot, p0))
            if n < 16:      # decoded tokens and short portions: plain lists (an array per field would cost more than it saves)
                ids.append([int(t) for t in toks])
                row_slot.append([slot] * n)
                row_pos.append(list(range(p0, p0 + n)))
                row_prev.append([-1] + list(range(r0, r0 + n - 1)))
            else:
                ids.append(np.asarray(toks, dtype=np.int32))
                row_slot.append(np.full(n, slot, dtype=np.int32))
                row_pos.append(np.arange(p0, p0 + n, dtype=np.int32))
                prev = np.arange(r0 - 1, r0 + n - 1, dtype=np.int32)
                prev[0] = -1
                row_prev.append(prev)
            r0 += n
        def flat(pieces):
            if all(isinstance(a, list) for a in pieces):
                return [v for a in pieces for v in a]
            return np.concatenate([np.asarray(a, dtype=np.int32) for a in pieces])
        ids, row_slot, row_pos, row_prev = flat(ids), flat(row_slot), flat(row_pos), flat(row_prev)
        return RaggedBatch(ids, row_slot, row_pos, row_prev, seq_start, seq_len, seq_slot, portions, self.device)
