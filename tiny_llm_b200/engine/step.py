"""The step function: one batch of (request, its next tokens) -- portions of prompts beside single
decoded tokens, cut anywhere -- runs as ONE batch from the cache and returns the logits at the
wanted places.

The reference runs either whole prompts or one token per request, switched by a global flag, and
rebuilds and uploads a block table per layer with a stream synchronisation each
(tiny_llm/runtime/cuda/cuda_runtime.cpp:658-802).  Here every step's metadata is laid out in one
pinned host buffer and goes to the device in one copy:

  tokens[T] positions[T] token_request[T] | cu_q[R+1] q_start[R] kv_len[R] slot[R] | logit_rows[n]
  | per cache group: slot_mapping[T], block_table[R, max_blocks]

A token's position is the number of tokens its request held before it; key j is visible to it iff
j <= position, whatever mix of portions and decoded tokens the batch has."""
from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache import CacheManager
from .workspace import Workspace


class OutOfPages(RuntimeError):
    """The cache cannot hold the step's new tokens; nothing was taken."""


@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()  # places among `tokens` whose logits are wanted


@dataclass
class KVView:
    """What a mixer with a KVNeed gets: its entry's pages and the step's tables of its group."""
    k: torch.Tensor              # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
    block_table: torch.Tensor    # int32 [R, max_blocks], -1 where a page was given back
    slot_mapping: torch.Tensor   # int32 [T]: page * page_size + offset of every token of the step
    page_size: int


@dataclass
class StateView:
    """What a mixer with a StateNeed gets: state[slot] is the request's state."""
    state: torch.Tensor          # [max_slots, *shape]


@dataclass
class GroupMeta:
    block_table: torch.Tensor
    slot_mapping: torch.Tensor
    max_blocks: int


@dataclass
class StepBatch:
    num_tokens: int
    num_requests: int
    num_logits: int
    tokens: torch.Tensor
    positions: torch.Tensor
    token_request: torch.Tensor
    cu_q: torch.Tensor
    q_start: torch.Tensor
    kv_len: torch.Tensor
    slots: torch.Tensor
    logit_rows: torch.Tensor
    groups: List[GroupMeta]
    max_q_len: int
    max_kv_len: int
    # host copies for parts that plan on the host
    host_q_lens: List[int] = field(default_factory=list)
    host_kv_lens: List[int] = field(default_factory=list)
    num_leading_decodes: int = 0   # how many requests at the front of the batch bring exactly one token


class StepContext:
    def __init__(self, runner: "ModelRunner", batch: StepBatch):
        self.runner = runner
        self.batch = batch
        self.dtype = runner.dtype
        self.device = runner.device
        self.workspace = runner.workspace

    def cache_view(self, order_pos: int):
        ref = self.runner.cache.refs[order_pos]
        if ref.group is not None:
            g = self.runner.cache.groups[ref.group]
            m = self.batch.groups[ref.group]
            return KVView(g.kv[ref.entry, 0], g.kv[ref.entry, 1], m.block_table, m.slot_mapping, g.page_size)
        if ref.state is not None:
            return StateView(self.runner.cache.slots.tensors[ref.state])
        return None


class ModelRunner:
    """Owns the model's device side: weights, cache storage, workspace, and the step function."""

    def __init__(self, model, cache: CacheManager, dtype: torch.dtype, device,
                 max_tokens_per_step: int = 8192, max_requests_per_step: int = 256):
        if not model.loaded:
            raise RuntimeError("the model has no weights yet")
        self.model = model
        self.cache = cache
        self.dtype = dtype
        self.device = torch.device(device)
        self.max_tokens_per_step = max_tokens_per_step
        self.max_requests_per_step = max_requests_per_step
        self.workspace = Workspace(self.device)
        self.max_blocks = -(-model.spec.max_positions // cache.page_size)
        t, r, g = max_tokens_per_step, max_requests_per_step, len(cache.groups)
        # fixed offsets (in int32 words) of every region of the metadata buffer
        self._off = {}
        cur = 0
        for name, n in (("tokens", t), ("positions", t), ("token_request", t), ("cu_q", r + 1),
                        ("q_start", r), ("kv_len", r), ("slots", r), ("logit_rows", t)):
            self._off[name] = (cur, n)
            cur += n
        for gi in range(g):
            self._off[f"slot_mapping{gi}"] = (cur, t)
            cur += t
        for gi in range(g):
            self._off[f"block_table{gi}"] = (cur, r * self.max_blocks)
            cur += r * self.max_blocks
        cur += 4 * (10 + 2 * g)      # room for the 16-byte alignment of the packed layout of one-token steps
        self._meta_words = cur
        # The host side of the metadata is a ring of pinned buffers: the copy to the device is
        # asynchronous, and a caller that enqueues steps without waiting for them must not overwrite a
        # buffer whose copy has not run yet.  An event per buffer says when its copy is done.
        pin = self.device.type == "cuda"
        self._staging = [torch.zeros(cur, dtype=torch.int32, pin_memory=pin) for _ in range(4 if pin else 1)]
        self._staging_done = [None] * len(self._staging)
        self._staging_next = 0
        self._dev_meta = torch.zeros(cur, dtype=torch.int32, device=self.device)
        self.steps_run = 0
        # CUDA graphs of decode-only steps, keyed by what is baked into their launches
        self.use_graphs = self.device.type == "cuda" and getattr(model, "graph_safe", False)
        self._graphs = {}
        self._graph_seen = set()
        self._table_rows = {}
        self._decode_layouts = {}
        self.last_h2d_bytes = 0     # bytes of the last step's metadata copy to the device
        self.graph_replays = 0
        # Tapes of the launches of all other steps, keyed by what their launches depend on; a step with a key seen
        # before runs its tape again instead of the model's Python code (a quarter of the host time per launch)
        self.use_tapes = self.use_graphs and os.environ.get("TLLM_TAPES", "1") != "0"
        self._tapes = {}
        self.tape_replays = 0

    # ---- metadata
    def _region(self, buf, name, n=None):
        off, cap = self._off[name]
        return buf[off: off + (cap if n is None else n)]

    def validate(self, entries: Sequence[StepEntry]) -> None:
        """Everything that can be wrong with a step is found before a page is taken."""
        cache = self.cache
        r = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        t = sum(q_lens)
        if r == 0 or t == 0:
            raise ValueError("a step needs at least one request with at least one token")
        if any(n == 0 for n in q_lens):
            raise ValueError("every request of a step brings at least one token")
        if t > self.max_tokens_per_step or r > self.max_requests_per_step:
            raise ValueError(f"step of {t} tokens / {r} requests exceeds the runner's limits "
                             f"({self.max_tokens_per_step} / {self.max_requests_per_step})")
        if len({e.rid for e in entries}) != r:
            raise ValueError("a request appears twice in one step")
        vocab = self.model.spec.vocab_size
        for e, n in zip(entries, q_lens):
            if not cache.has_request(e.rid):
                raise KeyError(f"request {e.rid!r} is not live in the cache")
            s = cache.kv_len[e.rid]
            if s + n > self.model.spec.max_positions:
                raise ValueError(f"request {e.rid!r} would reach {s + n} tokens; the model's limit is "
                                 f"{self.model.spec.max_positions}")
            if min(e.tokens) < 0 or max(e.tokens) >= vocab:
                raise ValueError(f"request {e.rid!r}: token id outside [0, {vocab})")
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.rid!r}: wanted place {w} is outside its {n} tokens")

    def build_batch(self, entries: Sequence[StepEntry], device_tokens=None) -> StepBatch:
        cache = self.cache
        r = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        t = sum(q_lens)
        starts = [cache.kv_len[e.rid] for e in entries]
        slot = self._staging_next
        self._staging_next = (slot + 1) % len(self._staging)
        if self._staging_done[slot] is not None:
            self._staging_done[slot].synchronize()   # the copy that last read this buffer has finished
        host_meta = self._staging[slot]
        host = host_meta.numpy()
        if t == r:
            return self._build_decode_batch(entries, starts, host_meta, host, slot, device_tokens)
        if device_tokens is not None:
            raise ValueError("token ids can stay on the device only in a step where every request brings one token")
        tok = self._region(host, "tokens", t)
        pos = self._region(host, "positions", t)
        req = self._region(host, "token_request", t)
        cu = self._region(host, "cu_q", r + 1)
        rows: List[int] = []
        cur = 0
        cu[0] = 0
        for i, (e, s, n) in enumerate(zip(entries, starts, q_lens)):
            tok[cur: cur + n] = np.asarray(e.tokens, dtype=np.int64)
            pos[cur: cur + n] = np.arange(s, s + n)
            req[cur: cur + n] = i
            rows.extend(cur + w for w in e.want)
            cur += n
            cu[i + 1] = cur
        self._region(host, "q_start", r)[:] = starts
        kv_after = [s + n for s, n in zip(starts, q_lens)]
        self._region(host, "kv_len", r)[:] = kv_after
        self._region(host, "slots", r)[:] = [cache.slot_of(e.rid) for e in entries]
        n_out = len(rows)
        if n_out:
            self._region(host, "logit_rows", n_out)[:] = rows
        max_blocks = self.max_blocks
        used_words = self._off["logit_rows"][0] + self._off["logit_rows"][1]
        group_hosts = []
        for gi, g in enumerate(cache.groups):
            sm = self._region(host, f"slot_mapping{gi}", t)
            bt = self._region(host, f"block_table{gi}", r * max_blocks).reshape(r, max_blocks)
            cur = 0
            for i, (e, s, n) in enumerate(zip(entries, starts, q_lens)):
                table = cache.block_table(gi, e.rid)
                nb = len(table)
                bt[i, :nb] = table
                bt[i, nb:] = -1
                p = np.arange(s, s + n)
                pages = np.asarray(table, dtype=np.int64)[p // g.page_size]
                if (pages < 0).any():
                    raise RuntimeError(f"request {e.rid!r} writes into a page it has given back")
                sm[cur: cur + n] = pages * g.page_size + p % g.page_size
                cur += n
            group_hosts.append((sm, bt))
            used_words = self._off[f"block_table{gi}"][0] + r * max_blocks
        # one copy, host to device
        self.last_h2d_bytes = 4 * used_words
        self._dev_meta[:used_words].copy_(host_meta[:used_words], non_blocking=True)
        if self.device.type == "cuda":
            if self._staging_done[slot] is None:
                self._staging_done[slot] = torch.cuda.Event()
            self._staging_done[slot].record()
        dev = self._dev_meta
        groups = []
        for gi in range(len(cache.groups)):
            groups.append(GroupMeta(
                block_table=self._region(dev, f"block_table{gi}", r * max_blocks).view(r, max_blocks),
                slot_mapping=self._region(dev, f"slot_mapping{gi}", t), max_blocks=max_blocks))
        return StepBatch(
            num_tokens=t, num_requests=r, num_logits=n_out,
            tokens=self._region(dev, "tokens", t), positions=self._region(dev, "positions", t),
            token_request=self._region(dev, "token_request", t), cu_q=self._region(dev, "cu_q", r + 1),
            q_start=self._region(dev, "q_start", r), kv_len=self._region(dev, "kv_len", r),
            slots=self._region(dev, "slots", r), logit_rows=self._region(dev, "logit_rows", n_out),
            groups=groups, max_q_len=max(q_lens), max_kv_len=max(kv_after),
            host_q_lens=q_lens, host_kv_lens=kv_after,
            num_leading_decodes=next((i for i, n in enumerate(q_lens) if n != 1), r))

    def _table_row(self, gi: int, rid, table: List[int]) -> np.ndarray:
        """The request's block table as a cached int32 row of max_blocks entries (-1 beyond its pages)."""
        key = (gi, rid)
        held = self._table_rows.get(key)
        if held is None:
            if len(self._table_rows) > 8 * self.max_requests_per_step:   # rows of requests that have ended
                live = {(g, rid2) for g in range(len(self.cache.groups)) for rid2 in self.cache.kv_len}
                self._table_rows = {k: v for k, v in self._table_rows.items() if k in live}
            held = [np.full(self.max_blocks, -1, dtype=np.int32), 0, -1]
            self._table_rows[key] = held
        row, n, birth = held
        if birth != self.cache.birth[rid]:   # another life of this request id: its pages are others
            row[:] = -1
            n = 0
            held[2] = self.cache.birth[rid]
        if n != len(table):
            row[n: len(table)] = table[n:]
            held[1] = len(table)
        return row

    def _decode_layout(self, r: int):
        """Where the regions lie in a step of r one-token requests: the same order as the general layout, but
        sized for r and packed from the start of the buffer (each region on a 16-byte boundary), so that the
        copy to the device is as long as the step's own tables and not as the largest step's.  The layout
        depends on r alone, which is also what a captured graph of such a step is keyed by."""
        lay = self._decode_layouts.get(r)
        if lay is None:
            lay, cur = {}, 0
            names = [("tokens", r), ("positions", r), ("token_request", r), ("cu_q", r + 1), ("q_start", r), ("kv_len", r),
                     ("slots", r), ("logit_rows", r)]
            names += [(f"slot_mapping{gi}", r) for gi in range(len(self.cache.groups))]
            names += [(f"block_table{gi}", r * self.max_blocks) for gi in range(len(self.cache.groups))]
            for name, n in names:
                lay[name] = (cur, n)
                cur += -(-n // 4) * 4
            lay["_words"] = cur
            self._decode_layouts[r] = lay
        return lay

    def _build_decode_batch(self, entries, starts, host_meta, host, slot, device_tokens=None) -> StepBatch:
        """The common step: every request brings one token.  Filled with whole-array writes; block tables
        come from rows cached per request; the regions are packed (see _decode_layout)."""
        cache = self.cache
        r = len(entries)
        lay = self._decode_layout(r)

        def region(buf, name, n=None):
            off, cap = lay[name]
            return buf[off: off + (cap if n is None else n)]

        starts_np = np.asarray(starts, dtype=np.int64)
        region(host, "tokens")[:] = [e.tokens[0] for e in entries]
        region(host, "positions")[:] = starts_np
        region(host, "token_request")[:] = np.arange(r)
        region(host, "cu_q")[:] = np.arange(r + 1)
        region(host, "q_start")[:] = starts_np
        region(host, "kv_len")[:] = starts_np + 1
        region(host, "slots")[:] = [cache.slot_of(e.rid) for e in entries]
        rows = [i for i, e in enumerate(entries) if len(e.want)]
        n_out = len(rows)
        if n_out:
            region(host, "logit_rows", n_out)[:] = rows
        max_blocks = self.max_blocks
        for gi, g in enumerate(cache.groups):
            sm = region(host, f"slot_mapping{gi}")
            bt = region(host, f"block_table{gi}").reshape(r, max_blocks)
            windowed = g.need.window is not None
            for i, e in enumerate(entries):
                table = cache.block_table(gi, e.rid)
                if windowed:     # entries of a windowed group turn to -1 as the window moves: no cached row
                    bt[i, :len(table)] = table
                    bt[i, len(table):] = -1
                else:
                    bt[i] = self._table_row(gi, e.rid, table)
            blocks = starts_np // g.page_size
            pages = bt[np.arange(r), blocks].astype(np.int64)
            if (pages < 0).any():
                raise RuntimeError("a request writes into a page it has given back")
            sm[:] = pages * g.page_size + starts_np % g.page_size
        used_words = lay["_words"]
        self.last_h2d_bytes = 4 * used_words
        self._dev_meta[:used_words].copy_(host_meta[:used_words], non_blocking=True)
        if self.device.type == "cuda":
            if self._staging_done[slot] is None:
                self._staging_done[slot] = torch.cuda.Event()
            self._staging_done[slot].record()
        dev = self._dev_meta
        if device_tokens is not None:   # the ids were chosen on the device and have not been to the host yet
            region(dev, "tokens").copy_(device_tokens[:r], non_blocking=True)
        groups = [GroupMeta(block_table=region(dev, f"block_table{gi}").view(r, max_blocks),
                            slot_mapping=region(dev, f"slot_mapping{gi}"), max_blocks=max_blocks)
                  for gi in range(len(cache.groups))]
        kv_after = [s + 1 for s in starts]
        return StepBatch(
            num_tokens=r, num_requests=r, num_logits=n_out,
            tokens=region(dev, "tokens"), positions=region(dev, "positions"),
            token_request=region(dev, "token_request"), cu_q=region(dev, "cu_q"),
            q_start=region(dev, "q_start"), kv_len=region(dev, "kv_len"),
            slots=region(dev, "slots"), logit_rows=region(dev, "logit_rows", n_out),
            groups=groups, max_q_len=1, max_kv_len=max(kv_after), host_q_lens=[1] * r, host_kv_lens=kv_after)

    # ---- the step
    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs exactly the tokens it is given, as one batch, from the cache earlier steps left.
        Returns float32 logits [number of wanted places, vocab] in the order of the entries and of
        their `want` lists, or None if nothing is wanted.  The returned tensor is workspace memory:
        it is valid until the next step.
        `device_tokens` (int32 on the device, one id per entry, entries of one token each): the ids to
        run instead of the entries' own, for a caller that chains steps without reading the sampled
        ids back first."""
        cache = self.cache
        self.validate(entries)
        need = [0] * len(cache.groups)
        for e in entries:
            for gi, m in enumerate(cache.pages_missing(e.rid, len(e.tokens))):
                need[gi] += m
        if any(n > g.pool.num_free for n, g in zip(need, cache.groups)):
            raise OutOfPages(f"the step needs {need} new pages per cache group, "
                             f"free: {[g.pool.num_free for g in cache.groups]}")
        for e in entries:
            ok = cache.reserve(e.rid, len(e.tokens))
            assert ok
        batch = self.build_batch(entries, device_tokens)
        logits = self._run(entries, batch)
        for e in entries:
            cache.commit(e.rid, len(e.tokens))
        self.steps_run += 1
        return logits

    # ---- launch: eagerly, or as the replay of a captured graph when the step only decodes
    def _graph_key(self, entries, batch: StepBatch):
        """Steps in which every request brings one token and wants its logits replay a CUDA graph.
        Baked into a graph: the number of requests and the bucket of the longest context (it fixes
        how attention slices the keys); everything else is read from the metadata on the device."""
        if not self.use_graphs or batch.max_q_len != 1 or batch.num_logits != batch.num_requests:
            return None
        if any(len(e.want) != 1 for e in entries):
            return None
        bucket = 256
        while bucket < batch.max_kv_len:
            bucket *= 2
        return (batch.num_requests, bucket)

    def _tape_key(self, batch: StepBatch):
        """What the launches of a step are made from on the host: the numbers of tokens, requests and wanted places,
        the longest portion, the bucket of the longest context (it fixes how attention slices the keys), how many
        requests at the front bring one token (attention runs those apart), the stream and the kernel switches.  All else (ids, positions, tables, slots) the kernels read from device memory at
        addresses that do not move."""
        if not self.use_tapes:
            return None
        bucket = 256
        while bucket < batch.max_kv_len:
            bucket *= 2
        return (batch.num_tokens, batch.num_requests, batch.num_logits, batch.max_q_len, bucket,
                batch.num_leading_decodes, torch.cuda.current_stream(self.device).cuda_stream, ops.knobs())

    MAX_TAPES = 64

    def _run_taped(self, batch: StepBatch):
        key = self._tape_key(batch)
        if key is None:
            return self.model.forward(StepContext(self, batch))
        batch.max_kv_len = key[4]
        held = self._tapes.get(key)
        if held is not None:
            ops.replay_tape(held[0])
            self.tape_replays += 1
            return held[1]
        ops.begin_tape()
        try:
            logits = self.model.forward(StepContext(self, batch))
        finally:
            tape = ops.end_tape()
        if len(self._tapes) >= self.MAX_TAPES:
            self._tapes.pop(next(iter(self._tapes)))     # the oldest
        # the tape's launches point into these buffers: keep them alive even if the workspace grows
        self._tapes[key] = (tape, logits, list(self.workspace._buffers.values()))
        return logits

    def _run(self, entries, batch: StepBatch):
        key = self._graph_key(entries, batch)
        if key is None:
            return self._run_taped(batch)
        batch.max_kv_len = key[1]
        held = self._graphs.get(key)
        if held is None:
            if key not in self._graph_seen:
                # first time: run eagerly (this also sizes the workspace and configures the kernels)
                self._graph_seen.add(key)
                return self.model.forward(StepContext(self, batch))
            graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize(self.device)
            before = ops.launches
            with torch.cuda.graph(graph):
                logits = self.model.forward(StepContext(self, batch))
            kernels = ops.launches - before
            ops.launches = before
            # the graph's launches point into these buffers: keep them alive even if the workspace grows
            held = (graph, logits, list(self.workspace._buffers.values()), kernels)
            self._graphs[key] = held
        held[0].replay()
        ops.launches += held[3]
        self.graph_replays += 1
        return held[1]
