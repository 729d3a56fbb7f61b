"""Step function, cache and state manager for models built from the ragged-token-batch mechanisms (``layers``).

``SequenceEngine`` owns, for every layer run of a model, what that run's mixer declares in ``state_spec``: page pools for softmax
attention (pages handed out by the same bookkeeping as the batched Llama decoder, ``batch.KvPages``) and slot-indexed fp32 state for the
recurrent mixers; a layer may also borrow state another layer owns (``"borrow"`` in its ``state_spec``: attention over an earlier
layer's cache), and the engine keeps each request's last token for models whose embedding looks at the previous one. One ``run`` is one step: any mix of portions of prompts and single decoded tokens, each request at its own position.
Logits at a position do not depend on how the tokens were cut into steps, on the neighbours in the batch, or on which pages and slot a
request got, beyond the rounding of differently ordered sums.

``SequenceDecoder`` puts the decoder interface of ``scheduler.ContinuousBatcher`` on top (add / step / tokens / remove / position ...),
with prompts processed in chunks beside the decoding requests and the device sampler (``sllm_sample_f32``) for the next tokens.

Additive to the reference, which decodes one sequence token by token (source/model/model.cpp:148-185)."""
from __future__ import annotations

import gc
import weakref

import numpy as np
import torch

from . import _lib
from .batch import KvPages
from .config import BF16

QUERY_TILE = 32      # queries per attention work item (kBQ of csrc/seq_attn.cu)
KEY_TILE = 32


class Step:
    """What the mechanisms see of one step: sizes, the batch description, the stream, scratch memory."""

    def __init__(self, engine):
        # no strong reference back: an engine must die with its last user (by reference count), not whenever the cycle collector runs —
        # its captured graphs free device memory when they go, and that is not allowed while another engine is capturing a step
        self.engine = weakref.proxy(engine)
        self.T = self.nseg = 0
        self.b = _lib.SeqBatch()
        self.st = None
        self.nsplit = 1
        self.prev_ids = None      # device array [T]: the token before each token in its sequence, -1 at a sequence's start

    def scratch(self, name: str, n_floats: int) -> torch.Tensor:
        return self.engine._scratch(name, n_floats)

    def gemm_scratch(self, K: int, N: int):
        """bf16 copy of the activations + the plain product, for products that go to the tensor cores (None: too few rows to pay)."""
        if not self.engine.tensor_cores or self.T < 64:
            return None
        n_bytes = ((self.T * K * 2 + 255) // 256) * 256 + self.T * N * 4
        return self.engine._scratch("gemm", (n_bytes + 3) // 4)


class SequenceEngine:
    def __init__(self, model, max_tokens: int, max_seqs: int = 4, page_len: int = 64, tensor_cores: bool | None = None, graphs: bool = True):
        if page_len % KEY_TILE:
            raise ValueError(f"page_len must be a multiple of {KEY_TILE}")
        self.model, self.ops, self.device = model, model.ops, model.device
        self.max_seqs, self.page_len = max_seqs, page_len
        self.n_pages = max(1, -(-max_tokens // page_len))
        self.max_pages = self.n_pages                       # one request may hold the whole pool
        self.max_len = self.n_pages * page_len
        self.pages = KvPages(self.n_pages, page_len, max_seqs, self.max_pages)
        self.tensor_cores = self.ops.tensor_cores if tensor_cores is None else (tensor_cores and self.ops.w_dtype == BF16)
        kv_t = torch.bfloat16 if self.ops.kv_dtype == BF16 else torch.float32
        self.states = []
        for spec in model.state_specs():
            st = {}
            for name, kv_heads, width in spec["pages"]:
                st[name] = torch.zeros(self.n_pages, kv_heads, page_len, width, dtype=kv_t, device=self.device)
            for name, shape in spec["slots"]:
                st[name] = torch.zeros((max_seqs,) + tuple(shape), dtype=torch.float32, device=self.device)
            self.states.append(st)
        # a layer may read state that another layer run owns (attention over an earlier layer's cache): one memory, two names
        for st, spec in zip(self.states, model.state_specs()):
            for name, run, src in spec.get("borrow", []):
                if not 0 <= run < len(self.states) or src not in self.states[run]:
                    raise ValueError(f"state {name!r} is borrowed from layer run {run}, which has no {src!r}")
                st[name] = self.states[run][src]
        self._slot_tensors = [t for st, spec in zip(self.states, model.state_specs()) for name, _ in spec["slots"] for t in [st[name]]]
        self.free_slots = list(range(max_seqs - 1, -1, -1))
        self.pos = [0] * max_seqs
        self.last_token = [-1] * max_seqs       # the token at position pos - 1 of each request (-1: none yet), part of its state
        self.live = set()
        self._bufs = {}
        self._meta_dev = None
        self._meta_host = None
        self._meta_event = None
        self.step_obj = Step(self)
        self.steps_run = 0
        # Steps of single tokens (decoding) are launch-bound: their kernel sequence depends only on how many requests step and how many
        # rows of logits are asked for (tokens, positions, slots and the block table are device memory), so it is captured once per such
        # pair as a CUDA graph and replayed. The first step of a kind runs directly (it sizes the scratch buffers), the second is captured.
        self.graphs = graphs and self.device.type == "cuda"
        self._graphs = {}
        self.graph_replays = 0

    # ---- requests ----
    def admit(self) -> int:
        """A free state slot for a new request; its recurrent state starts at zero."""
        if not self.free_slots:
            raise RuntimeError(f"all {self.max_seqs} state slots are in use")
        slot = self.free_slots.pop()
        for t in self._slot_tensors:
            t[slot].zero_()
        self.pos[slot] = 0
        self.last_token[slot] = -1
        self.live.add(slot)
        return slot

    def release(self, slot: int) -> None:
        """Give back the request's pages and its slot."""
        if slot not in self.live:
            raise ValueError(f"slot {slot} is not in use")
        self.pages.release(slot)
        self.live.discard(slot)
        self.free_slots.append(slot)

    @property
    def free_pages(self) -> int:
        return self.pages.free

    # ---- memory ----
    def _scratch(self, name: str, n_floats: int) -> torch.Tensor:
        t = self._bufs.get(name)
        if t is None or t.numel() < n_floats:
            t = torch.empty(max(n_floats, 1), dtype=torch.float32, device=self.device)
            self._bufs[name] = t
            self._graphs = {}          # captured steps hold the old address
        return t

    def _upload(self, arrays):
        """The step's index arrays as ONE host-to-device copy; returns their device addresses."""
        sizes = [a.size for a in arrays]
        total = sum(sizes)
        if self._meta_host is None or self._meta_host.numel() < total:
            # sized once for the largest step the pool can hold, so that the addresses captured in graphs stay valid
            cap = max(total, 6 * self.max_len + 16 * self.max_seqs + self.max_seqs * self.max_pages + 64)
            self._graphs = {}
            self._meta_host = torch.empty(cap, dtype=torch.int32).pin_memory() if self.device.type == "cuda" else torch.empty(cap, dtype=torch.int32)
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        if self._meta_event is not None:
            self._meta_event.synchronize()          # the previous step's copy has left the pinned buffer
        host = self._meta_host.numpy()
        off, ptrs = 0, []
        for a, n in zip(arrays, sizes):
            host[off:off + n] = a.reshape(-1)
            ptrs.append(self._meta_dev.data_ptr() + 4 * off)
            off += n
        self._meta_dev[:total].copy_(self._meta_host[:total], non_blocking=True)
        if self.device.type == "cuda":
            self._meta_event = torch.cuda.Event()
            self._meta_event.record()
        return ptrs

    # ---- the step ----
    def run(self, entries, tap=None):
        """entries: [(slot, tokens, want)] — for each request its next tokens and the indices among them whose logits are asked for.
        Returns a float32 tensor [sum of wants][vocab] on the device (None if nothing is wanted), rows in the order of entries and want."""
        entries = [(s, np.ascontiguousarray(t, dtype=np.int32).reshape(-1), list(w)) for s, t, w in entries]
        entries = [e for e in entries if e[1].size]
        if not entries:
            return None
        if len({s for s, _, _ in entries}) != len(entries):
            raise ValueError("a request may bring one portion per step")
        for slot, toks, _ in entries:                     # pages first, all or nothing
            if slot not in self.live:
                raise ValueError(f"slot {slot} is not in use")
        need = sum(max(0, -(-(self.pos[s] + t.size) // self.page_len) - self.pages.held(s)) for s, t, _ in entries)
        if need > self.pages.free:
            raise _lib.SllmError(_lib.ENOMEM, f"out of cache pages: this step needs {need} more, {self.pages.free} free")
        for slot, toks, _ in entries:
            self.pages.reserve(slot, self.pos[slot] + toks.size)
        T = sum(t.size for _, t, _ in entries)
        nseg = len(entries)
        ids = np.concatenate([t for _, t, _ in entries])
        prev_ids = np.concatenate([np.concatenate([[self.last_token[s]], t[:-1]]) for s, t, _ in entries]).astype(np.int32)
        tok_slot = np.concatenate([np.full(t.size, s, dtype=np.int32) for s, t, _ in entries])
        tok_pos = np.concatenate([np.arange(self.pos[s], self.pos[s] + t.size, dtype=np.int32) for s, t, _ in entries])
        seg_len = np.array([t.size for _, t, _ in entries], dtype=np.int32)
        seg_start = np.concatenate([[0], np.cumsum(seg_len)[:-1]]).astype(np.int32)
        seg_slot = np.array([s for s, _, _ in entries], dtype=np.int32)
        seg_pos0 = np.array([self.pos[s] for s, _, _ in entries], dtype=np.int32)
        seg_tile0 = np.concatenate([[0], np.cumsum(-(-seg_len // QUERY_TILE))[:-1]]).astype(np.int32)
        qt_seg, qt_off = [], []
        for i, n in enumerate(seg_len):
            for off in range(0, int(n), QUERY_TILE):
                qt_seg.append(i)
                qt_off.append(off)
        # long tiles first: a tile's work grows with its last position
        order = sorted(range(len(qt_seg)), key=lambda j: -(int(seg_pos0[qt_seg[j]]) + qt_off[j]))
        qt_seg = np.array([qt_seg[j] for j in order], dtype=np.int32)
        qt_off = np.array([qt_off[j] for j in order], dtype=np.int32)
        rows = np.array([int(seg_start[i]) + int(k) for i, (_, t, w) in enumerate(entries) for k in w], dtype=np.int32)
        for i, (_, t, w) in enumerate(entries):
            if any(k < 0 or k >= t.size for k in w):
                raise ValueError("a wanted index lies outside the entry's tokens")
        table = self.pages.table().astype(np.int32)
        arrays = [ids, tok_slot, tok_pos, seg_start, seg_len, seg_slot, seg_pos0, qt_seg, qt_off, rows if rows.size else np.zeros(1, np.int32), table, seg_tile0, prev_ids]
        p = self._upload(arrays)
        step = self.step_obj
        step.T, step.nseg = T, nseg
        b = step.b
        b.T, b.nseg = T, nseg
        b.tok_slot, b.tok_pos, b.seg_start, b.seg_len, b.seg_slot, b.seg_pos0 = p[1], p[2], p[3], p[4], p[5], p[6]
        b.qt_seg, b.qt_off, b.n_qtiles = p[7], p[8], int(qt_seg.size)
        b.block_table, b.max_pages, b.page_len = p[10], self.max_pages, self.page_len
        b.seg_tile0 = p[11]
        step.prev_ids = _PtrView(p[12])
        ids_t = _PtrView(p[0])
        rows_t = _PtrView(p[9])
        n_rows = int(rows.size)
        decode_only = T == nseg
        if decode_only:
            # a fixed share count per batch size keeps the launch sequence of a decoding step independent of the context lengths
            step.nsplit = max(1, 32 // nseg)
        else:
            # share the key tiles of long contexts among CTAs when the step has few query tiles
            key_tiles = max(1, -(-int((seg_pos0 + seg_len).max()) // KEY_TILE))
            step.nsplit = int(min(key_tiles, max(1, 64 // max(1, int(qt_seg.size)))))
        key = (nseg, n_rows)
        if decode_only and self.graphs and tap is None and key in self._graphs:
            entry = self._graphs[key]
            if entry is None:                               # second step of this kind: capture it (a capture does not execute)
                meta_addr = self._meta_dev.data_ptr()
                g = torch.cuda.CUDAGraph()
                collecting = gc.isenabled()
                gc.disable()        # a finaliser that frees device memory (another engine's graphs, say) must not run inside the capture
                try:
                    with torch.cuda.graph(g):
                        step.st = torch.cuda.current_stream(self.device).cuda_stream
                        out = self.model.forward(step, ids_t, self.states, rows_t, n_rows)
                finally:
                    if collecting:
                        gc.enable()
                entry = self._graphs[key] = (g, out, meta_addr, p[0], p[9])
            g, logits, meta_addr, ids_addr, rows_addr = entry
            if meta_addr != self._meta_dev.data_ptr() or ids_addr != p[0] or rows_addr != p[9]:
                raise RuntimeError("the step's index arrays moved under a captured graph")
            g.replay()
            self.graph_replays += 1
        else:
            if decode_only and self.graphs and tap is None:
                self._graphs[key] = None                    # seen once: capture at the next one
            step.st = torch.cuda.current_stream(self.device).cuda_stream
            logits = self.model.forward(step, ids_t, self.states, rows_t, n_rows, tap=tap)
        for slot, toks, _ in entries:
            self.pos[slot] += int(toks.size)
            self.last_token[slot] = int(toks[-1])
        self.steps_run += 1
        return logits


class _PtrView:
    """A device address with the one method the launch wrappers use of a tensor."""

    def __init__(self, ptr: int):
        self._ptr = ptr

    def data_ptr(self) -> int:
        return self._ptr


class SequenceDecoder:
    """The decoder interface of ``scheduler.ContinuousBatcher`` over a ``SequenceEngine``: every ``step`` feeds each live request either its
    next portion of the prompt (at most ``prefill_chunk`` tokens) or its last produced token, and draws the next token of every request
    whose prompt is through. ``tokens(slot)`` follows the convention of the batched Llama decoder: the tokens that FOLLOWED positions
    0 .. position-1 (the prompt's own continuation first, then what was produced)."""

    def __init__(self, engine: SequenceEngine, prefill_chunk: int = 256):
        self.engine, self.prefill_chunk = engine, max(1, prefill_chunk)
        self.max_seqs, self.page_len, self.n_pages, self.max_len = engine.max_seqs, engine.page_len, engine.n_pages, engine.max_len
        self._req = {}
        self._idx = torch.zeros(engine.max_seqs, dtype=torch.int32, device=engine.device)

    @property
    def free_pages(self) -> int:
        return self.engine.free_pages

    def add(self, prompt) -> int:
        prompt = np.ascontiguousarray(prompt, dtype=np.int32).reshape(-1)
        if prompt.size < 1:
            raise ValueError("empty prompt")
        slot = self.engine.admit()
        self._req[slot] = {"prompt": prompt, "fed": 0, "out": [], "limit": None, "sampling": None}
        return slot

    def set_limit(self, slot: int, positions: int) -> None:
        """The request stops taking part in steps once it holds this many positions."""
        self._req[slot]["limit"] = int(positions)

    def set_sampling(self, slot: int, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0, seed: int = 0) -> None:
        self._req[slot]["sampling"] = (float(temperature), int(top_k), float(top_p), int(seed))

    def position(self, slot: int) -> int:
        return self.engine.pos[slot]

    def remove(self, slot: int) -> None:
        self.engine.release(slot)
        del self._req[slot]

    def tokens(self, slot: int) -> np.ndarray:
        r = self._req[slot]
        return np.concatenate([r["prompt"][1:r["fed"]], np.array(r["out"], dtype=np.int32)]).astype(np.int32)

    def step(self, n: int = 1) -> None:
        eng = self.engine
        for _ in range(n):
            entries, drawing = [], []
            for slot, r in self._req.items():
                if r["limit"] is not None and eng.pos[slot] >= r["limit"]:
                    continue
                left = r["prompt"].size - r["fed"]
                if left > 0:
                    take = min(left, self.prefill_chunk)
                    toks = r["prompt"][r["fed"]:r["fed"] + take]
                    r["fed"] += take
                    last = r["fed"] == r["prompt"].size
                    entries.append((slot, toks, [take - 1] if last else []))
                    if last:
                        drawing.append(slot)
                else:
                    entries.append((slot, np.array([r["out"][-1]], dtype=np.int32), [0]))
                    drawing.append(slot)
            if not entries:
                return
            logits = eng.run(entries)
            if not drawing:
                continue
            st = torch.cuda.current_stream(eng.device).cuda_stream
            for i, slot in enumerate(drawing):
                temperature, top_k, top_p, seed = self._req[slot]["sampling"] or (0.0, 0, 0.0, 0)
                eng.ops.sample(logits.data_ptr() + 4 * i * logits.shape[1], logits.shape[1], temperature, top_k, top_p, seed, eng.pos[slot] - 1,
                               self._idx.data_ptr() + 4 * i, st)
            drawn = self._idx[:len(drawing)].cpu().numpy()
            for i, slot in enumerate(drawing):
                self._req[slot]["out"].append(int(drawn[i]))
