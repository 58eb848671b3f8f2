"""Engine and Scheduler for the config-driven models (hybrid.HybridDecoder).

Engine.step(entries) is THE step function: every entry brings the next tokens of one request (a prompt portion of
any length, or one decoded token); all entries run as one ragged batch through the model from the K/V pages and state
slots earlier steps left.  A request is admitted (state slot) at its first entry, may sit out steps, and gives back its
slot and pages with `finish`.

Scheduler is continuous batching on top of it: waiting requests are admitted while slots and pool tokens last, prompts
are fed in chunks under a per-step token budget next to the running requests' single decode tokens, and the next token
of every request whose last fed token ended its prompt (or was a decoded token) is sampled on the device with the
framework's samplers (greedy pa_argmax_f32; temperature / top-k / top-p through llm_decoder.sampling)."""
import collections

import torch

from . import _cabi
from .host_stage import to_device as _to_device


class Engine:
    def __init__(self, model):
        self.model = model
        self.states = model.states
        self._slot = {}          # request id -> slot

    def live(self):
        return list(self._slot)

    def has(self, rid):
        return rid in self._slot

    def length(self, rid):
        return self.states.length(self._slot[rid])

    def step(self, entries):
        """entries: [(request id, token ids, wanted indices into these tokens)].  Returns float logits
        [total wanted, vocab] (device) in entry / wanted order."""
        batch_entries, want, row0 = [], [], 0
        for rid, toks, wanted in entries:
            if not len(toks):
                continue
            if rid not in self._slot:
                self._slot[rid] = self.states.alloc()
            batch_entries.append((self._slot[rid], toks))
            for w in wanted:
                if not 0 <= int(w) < len(toks):
                    raise ValueError("wanted index outside the entry's tokens")
                want.append(row0 + int(w))
            row0 += len(toks)
        dev = self.model.device
        if not batch_entries:
            return torch.empty((0, self.model.vocab), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            batch = self.states.make_batch(batch_entries)
            want_rows = _to_device(torch.tensor(want, dtype=torch.int32), dev)
            return self.model.forward(batch, want_rows)

    def finish(self, rid):
        slot = self._slot.pop(rid, None)
        if slot is not None:
            self.states.free(slot)


class _Request:
    def __init__(self, rid, prompt, max_new_tokens):
        self.rid, self.prompt, self.max_new = rid, list(prompt), int(max_new_tokens)
        self.fed = 0            # prompt tokens already given to the engine
        self.out = []           # generated tokens
        self.pending = None     # a sampled token not yet fed


class Scheduler:
    def __init__(self, engine, max_batch_tokens=2048, temperature=1.0, top_k=0, top_p=1.0, eos_token_id=-1, seed=0):
        self.engine = engine
        self.max_batch_tokens = int(max_batch_tokens)
        self.temperature, self.top_k, self.top_p = float(temperature), int(top_k), float(top_p)
        self.eos = int(eos_token_id)
        self.waiting = collections.deque()
        self.running = []
        self.done = {}
        self._next = 0
        self._gen = None
        if self.top_k > 0 or self.top_p < 1.0:
            self._gen = torch.Generator(device=engine.model.device)
            self._gen.manual_seed(int(seed))

    def add_request(self, prompt, max_new_tokens, rid=None):
        if not len(prompt):
            raise ValueError("empty prompt")
        rid = self._next if rid is None else rid
        self._next += 1
        self.waiting.append(_Request(rid, prompt, max_new_tokens))
        return rid

    def _tiles(self, n):
        ts = self.engine.states.tile_size
        return (n + ts - 1) // ts * ts

    def _sample(self, logits):
        """logits [n, vocab] float -> [n] int32 next ids, on the device."""
        n, V = logits.shape
        ids = torch.empty(n, dtype=torch.int32, device=logits.device)
        lib = _cabi.lib()
        if self._gen is None:
            _cabi.check(lib.pa_argmax_f32(logits.data_ptr(), n, V, 1.0, 1, ids.data_ptr(), _cabi.stream()), "pa_argmax_f32")
            return ids
        from . import sampling
        probs = sampling.softmax_temperature(logits.contiguous(), self.temperature)
        sampling.apply_topk_topp_filter(probs, self.top_k, self.top_p, -1, 0.0)
        u = torch.rand(n, device=logits.device, generator=self._gen)
        sampling.sample_from_probs(probs, u, out=ids)
        return ids

    def step(self):
        """One engine step.  Returns False when nothing is left to do."""
        st = self.engine.states
        # admit: a request needs a slot and room for its whole prompt and output (it is never evicted half-way)
        reserved = sum(self._tiles(len(r.prompt) + r.max_new) - self._tiles(self.engine.length(r.rid) if self.engine.has(r.rid) else 0)
                       for r in self.running)
        while self.waiting and len(self.running) < st.max_seqs:
            r = self.waiting[0]
            need = self._tiles(len(r.prompt) + r.max_new)
            if reserved + need > st.free_tokens():
                if not self.running:
                    raise RuntimeError("request does not fit the cache pool")
                break
            reserved += need
            self.running.append(self.waiting.popleft())
        if not self.running:
            return False
        budget = self.max_batch_tokens
        entries, owners = [], []
        for r in self.running:                      # decode tokens first: one each
            if r.pending is not None and budget > 0:
                entries.append((r.rid, [r.pending], [0]))
                owners.append(r)
                r.pending = None
                budget -= 1
        for r in self.running:                      # then prompt portions under what is left of the budget
            if r.fed < len(r.prompt) and budget > 0:
                n = min(budget, len(r.prompt) - r.fed)
                toks = r.prompt[r.fed:r.fed + n]
                r.fed += n
                budget -= n
                last = r.fed == len(r.prompt)
                entries.append((r.rid, toks, [n - 1] if last else []))
                if last:
                    owners.append(r)
        logits = self.engine.step(entries)
        if owners:
            ids = self._sample(logits).cpu().tolist()
            for r, t in zip(owners, ids):
                r.out.append(int(t))
                if len(r.out) >= r.max_new or int(t) == self.eos:
                    self.engine.finish(r.rid)
                    self.done[r.rid] = r.prompt + r.out
                    self.running.remove(r)
                else:
                    r.pending = int(t)
        return bool(self.running or self.waiting)

    def run(self):
        while self.step():
            pass
        return self.done


def generate(model, prompts, max_new_tokens, **kw):
    """Greedy (or sampled) generation of several prompts of any lengths through Engine + Scheduler; returns
    prompt + generated ids per prompt."""
    sch = Scheduler(Engine(model), **kw)
    rids = [sch.add_request(p, max_new_tokens) for p in prompts]
    done = sch.run()
    return [done[r] for r in rids]
