"""The step function: one batch of (request, its next tokens) through the model.

A step runs only the tokens it is given — portions of prompts beside single decoded
tokens, cut anywhere — as one ragged batch against the cache that earlier steps left,
and returns float32 logits at the wanted places.  The ragged layout (flat tokens plus
``req_indptr``) is the reference's (v10_triton_paged_gqa/scheduler.py:182-223); unlike
the reference, which runs whole prompts and single decode tokens as two separate
forwards (v10_triton_paged_gqa/engine.py:105-133), every entry here has a cached
length before it (``kv_before``) and any number of new tokens.

Per step the host builds ONE int32 block (tokens, positions, token->request map,
request offsets, cached lengths, slots, logit rows, one block table per cache group) in
pinned memory and copies it to the device once.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Hashable, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheError
from ..cache.storage import CacheStorage
from ..config.engine import EngineConfig
from ..parts.model import LayeredModel
from ..sampling import SampleSpec
from .. import ops

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class OutOfPages(CacheError):
    """A step needs more pages than are free."""


@dataclass
class StepEntry:
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()  # places among ``tokens`` whose logits are asked for
    sample: Optional[SampleSpec] = None  # sample a token from the logits of the last token


@dataclass
class StepResult:
    logits: Optional[torch.Tensor]  # float32 [wanted, vocab]: ``want`` rows, then sampled rows
    tokens: Optional[torch.Tensor]  # int32 [sampled entries], in the order of the entries


@dataclass
class PendingSum:
    """A sum into the float32 stream ``acc`` that a product left unfinished."""

    partials: torch.Tensor  # float32 [splits, tokens, width] in the shared workspace
    splits: int
    bias: Optional[torch.Tensor]
    acc: torch.Tensor


class StepContext:
    """Everything a part may read about the current step."""

    def __init__(self, runner: "ModelRunner"):
        self._runner = runner
        self.dtype: torch.dtype = runner.dtype
        self.device = runner.device
        self.num_tokens = 0
        self.num_requests = 0
        self.max_q_len = 0
        self.max_kv_len = 0
        self.decode_only = False
        # device int32 tensors
        self.tokens = self.positions = self.token_req = None
        self.req_indptr = self.kv_before = self.slots = self.logit_rows = None
        # host copies (numpy int32) for parts that plan on the host
        self.req_indptr_host = self.kv_before_host = self.slots_host = None
        self.plans: dict = {}  # per-step plans parts share across layers
        self._pending: Optional[PendingSum] = None  # see ``leave_pending``
        # sampling rows of the step (device), None when every sampled row is greedy
        self.num_sampled = 0
        self.sample_temperature = self.sample_seed = self.sample_counter = None

    # A product may leave its last sum into a stream unfinished (float32 partial sums in the
    # shared workspace) so that whoever reads the stream next completes it inside its own kernel.
    def leave_pending(self, partials, splits: int, bias, acc) -> None:
        """``acc`` still lacks the sum of ``splits`` partial results (+ ``bias``)."""
        self.flush_pending()
        self._pending = PendingSum(partials, splits, bias, acc)
        ops.workspace_holder = self

    def take_pending(self, acc) -> Optional["PendingSum"]:
        """The unfinished sum into this very ``acc``, if there is one; the caller completes it."""
        pending = self._pending
        if pending is None or pending.acc is not acc:
            return None
        self._pending = None
        ops.workspace_holder = None
        return pending

    def flush_pending(self) -> None:
        """Complete an unfinished sum into a stream (see ``leave_pending``)."""
        pending = self._pending
        if pending is not None:
            self._pending = None
            ops.workspace_holder = None
            ops.finish_accum_norm(pending.partials, pending.splits, pending.bias, pending.acc)

    def buffer(self, name: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        return self._runner.buffer(name, shape, dtype)

    def upload(self, values) -> torch.Tensor:
        """Copy a small int32 array a part planned on the host to the device (valid for
        this step only)."""
        return self._runner.upload_aux(values)


class ModelRunner:
    def __init__(self, model: LayeredModel, config: EngineConfig):
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA is required: the engine has no CPU path")
        self.model = model
        self.config = config.resolve(model.spec.max_position_embeddings)
        self.device = torch.device(config.device)
        self.dtype = TORCH_DTYPES[config.dtype]
        if model.dtype != self.dtype:
            raise ValueError(f"the model was loaded as {model.dtype}, the engine runs {self.dtype}")
        self.vocab_size = model.spec.vocab_size
        self.storage = CacheStorage(
            model.cache_needs(), config.kv_block_size, config.max_decode_slots, config.max_num_blocks,
            config.max_seq_len, self.device, self.dtype,
        )
        self.cache = self.storage.manager
        self.num_groups = len(self.storage.groups)
        # rows of the persistent scratch buffers: the token budget, and the largest padded decode
        # batch a captured graph runs (a buffer that grew later would leave earlier graphs with
        # freed addresses)
        largest_graph = self._bucket(min(config.max_decode_slots, self.GRAPH_BUCKETS[-1]))
        self.token_capacity = max(config.max_num_batched_tokens, config.max_decode_slots, largest_graph)
        self._buffers: dict[str, torch.Tensor] = {}
        # two pinned staging blocks used in turn, each guarded by the event of its last copy
        self._meta_host = [None, None]
        self._meta_np = [None, None]
        self._meta_event = [None, None]
        self._meta_dev: Optional[torch.Tensor] = None
        self._meta_turn = 0
        self._aux_offset = 0
        self._graphs: dict = {}
        self._last_graph_ids: Optional[list] = None  # requests of the last step, if it was a graph decode step
        # The slot records on the device (csrc/slots.cu): last token, position, sampling counter,
        # temperature and seed of every slot, and the block tables of all slots.  Captured decode
        # steps read and advance them; ``_synced`` says which slots' records the device has as the
        # host knows them: slot -> (request, position, counter, temperature, seed); ``_device_pages``
        # says how many entries of such a slot's table rows the device has.
        self._records: Optional[torch.Tensor] = None
        self._slot_tables: Optional[torch.Tensor] = None
        self._synced: dict = {}
        self._device_pages = np.zeros(config.max_decode_slots, dtype=np.int32)
        self.h2d_bytes_last_step = 0
        self._tokens_host = [None, None]
        self._tokens_event = [None, None]
        self._tokens_turn = 0
        self._graph_safe = all(getattr(block.mixer, "graph_safe", False) for block in model.blocks)
        self.steps_run = 0
        self.graph_steps = 0

    # ------------------------------------------------------------- workspace
    def buffer(self, name: str, shape: tuple, dtype: torch.dtype, exact: bool = False) -> torch.Tensor:
        """A persistent scratch tensor; the first dimension is rows of the step.  It is
        sized for the token budget at once (``exact``: for the rows asked) so that its
        address stays the same from step to step."""
        rows, rest = shape[0], tuple(shape[1:])
        key = f"{name}|{rest}|{dtype}"
        flat = self._buffers.get(key)
        if flat is None or flat.shape[0] < rows:
            capacity = rows if exact else max(rows, self.token_capacity)
            flat = torch.empty((capacity, *rest), device=self.device, dtype=dtype)
            self._buffers[key] = flat
        return flat[:rows]

    def _meta(self, words: int):
        """A pinned host block and the device block of one step's int32 metadata."""
        turn = self._meta_turn = self._meta_turn ^ 1
        if self._meta_event[turn] is not None:
            self._meta_event[turn].synchronize()  # its last copy has left the host block
        if self._meta_host[turn] is None or self._meta_host[turn].numel() < words:
            size = max(words, 1 << 14)
            self._meta_host[turn] = torch.empty(size, dtype=torch.int32, pin_memory=True)
            self._meta_np[turn] = self._meta_host[turn].numpy()
        if self._meta_dev is None or self._meta_dev.numel() < words:
            self._meta_dev = torch.empty(max(words, 1 << 14), dtype=torch.int32, device=self.device)
        return self._meta_np[turn], self._meta_dev

    def _upload_meta(self, words: int) -> None:
        turn = self._meta_turn
        self._meta_dev[:words].copy_(self._meta_host[turn][:words], non_blocking=True)
        if self._meta_event[turn] is None:
            self._meta_event[turn] = torch.cuda.Event()
        self._meta_event[turn].record()

    def upload_aux(self, values) -> torch.Tensor:
        """Room after the step's metadata, in the same pinned and device blocks."""
        values = np.asarray(values, dtype=np.int32).reshape(-1)
        turn = self._meta_turn
        start, count = self._aux_offset, values.size
        if start + count > self._meta_host[turn].numel():
            raise ValueError("the step's host-planned data does not fit the metadata block")
        self._meta_np[turn][start:start + count] = values
        self._meta_dev[start:start + count].copy_(self._meta_host[turn][start:start + count], non_blocking=True)
        self._meta_event[turn].record()
        self._aux_offset += count
        return self._meta_dev[start:start + count]

    # -------------------------------------------------------------- requests
    def admit(self, request_id: Hashable) -> int:
        slot = self.cache.admit(request_id)
        self._synced.pop(slot, None)
        if self.storage.states:
            self.storage.clear_slot(slot)
        return slot

    def finish(self, request_id: Hashable) -> None:
        self._synced.pop(self.cache.finish(request_id), None)
        self._last_graph_ids = None

    def reserve(self, request_id: Hashable, new_len: int) -> bool:
        """Pages for the request's tokens up to ``new_len``; False when a pool is short."""
        return self.cache.extend(request_id, new_len)

    # ------------------------------------------------------------------ step
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries as one batch.  Returns float32 logits ``[wanted, vocab]`` in
        the order of the entries and of their ``want`` (None if nothing is wanted).
        The tensor is reused by the next step."""
        return self.run(entries).logits

    def run(self, entries: Sequence[StepEntry], feed_previous: bool = False) -> StepResult:
        """Run the entries as one batch: logits at the wanted places and, for entries
        with ``sample`` set, a token sampled from the logits of their last token.
        Both tensors are reused by the next step.

        ``feed_previous``: the entries are the requests of the previous step, which was a
        decode step replayed from a graph, in the same order; each one's token is the one
        that step sampled, taken on the device (``tokens`` of the entries is ignored), so
        this step can be launched before the host has seen those tokens."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return StepResult(None, None)
        try:
            return self._run(entries, feed_previous)
        except BaseException:
            # a step that broke in the middle leaves nothing for the next one: no unfinished sum
            # waiting for a later kernel, no trust in the device's slot records
            ops.workspace_holder = None
            self._synced.clear()
            self._last_graph_ids = None
            raise

    def _run(self, entries, feed_previous: bool) -> StepResult:
        if feed_previous:
            if not self.can_feed_previous(entries):
                raise ValueError("feed_previous needs the previous step's requests, in its order, as a graph decode step")
            return self._run_decode_graph(entries, feed_previous=True)
        if self._graphable(entries):
            return self._run_decode_graph(entries)
        if self._graphable_for_logits(entries):
            # single tokens whose logits are asked for and nothing sampled (trace replay): the same
            # captured decode step; its sampling lane runs greedily and its token is not handed out
            sampled = [StepEntry(e.request_id, e.tokens, sample=SampleSpec(0.0, 0, self.cache.num_tokens(e.request_id)))
                       for e in entries]
            return StepResult(self._run_decode_graph(sampled).logits, None)
        self._last_graph_ids = None
        ctx, caches = self._build(entries)
        with torch.no_grad():
            acc = self.model.forward(ctx, caches)
            logits = tokens = None
            wanted = ctx.logit_rows.numel() if ctx.logit_rows is not None else 0
            if wanted:
                logits = self.buffer("logits", (wanted, self.vocab_size), torch.float32, exact=True)
                self.model.logits(ctx, acc, ctx.logit_rows, logits)
            if ctx.num_sampled:
                tokens = self.buffer("sampled", (ctx.num_sampled,), torch.int32)
                rows = logits[wanted - ctx.num_sampled:]
                if ctx.sample_temperature is None:
                    ops.sample(rows, tokens)
                else:
                    ops.sample(rows, tokens, ctx.sample_temperature, ctx.sample_seed, ctx.sample_counter)
        for e in entries:
            self.cache.advance(e.request_id, self.cache.num_tokens(e.request_id) + len(e.tokens))
            self._synced.pop(self.cache.slot_of(e.request_id), None)  # the device's record of the slot is behind
        self.steps_run += 1
        return StepResult(logits, tokens)

    # ------------------------------------------------------ decode by CUDA graph
    # A step in which every entry brings one token and samples is replayed from a CUDA
    # graph captured once per batch-size bucket over static buffers, as the reference
    # captures its decode forward (v10_triton_paged_gqa/engine.py:137-185).  Lanes beyond
    # the live requests are padding: token 0 at position 0 of the reserved page 0.
    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)

    def _graphable(self, entries) -> bool:
        if not self.config.cuda_graph or not self._graph_safe:
            return False
        if len(entries) > min(self.config.max_decode_slots, self.GRAPH_BUCKETS[-1]):
            return False
        return all(len(e.tokens) == 1 and e.sample is not None and not e.want for e in entries)

    def _graphable_for_logits(self, entries) -> bool:
        if not self.config.cuda_graph or not self._graph_safe:
            return False
        if len(entries) > min(self.config.max_decode_slots, self.GRAPH_BUCKETS[-1]):
            return False
        return all(len(e.tokens) == 1 and e.sample is None and list(e.want) == [0] for e in entries)

    def _bucket(self, n: int) -> int:
        for b in self.GRAPH_BUCKETS:
            if b >= n:
                return b
        raise ValueError(n)

    def _graph_layout(self, b: int):
        """Offsets (in int32 words) of the static block of bucket ``b``: first the command block
        the host writes every step (csrc/slots.cu), then the lane-indexed words the kernels read,
        which the first kernel of the graph fills from the slot records."""
        W, G = self.cache.max_pages_per_request, self.num_groups
        capacity = b * max(G, 1)  # table entries a step can add: one a lane and group
        command = ops.slot_command_words(b, capacity)
        names = (("command", command), ("pad0", command & 1), ("seed", 2 * b), ("tok", b), ("pos", b), ("req", b),
                 ("ind", b + 1), ("kvb", b), ("slot", b), ("row", b), ("temp", b), ("count", b))
        layout, o = {}, 0
        for name, size in names:
            layout[name] = (o, size)
            o += size
        layout["tables"] = [(o + g * b * W, b * W) for g in range(G)]
        layout["capacity"] = capacity
        return layout, o + G * b * W

    def _slot_records(self):
        if self._records is None:
            S, W, G = self.config.max_decode_slots, self.cache.max_pages_per_request, self.num_groups
            self._records = torch.zeros((ops.slot_record_rows(), S), dtype=torch.int32, device=self.device)
            self._slot_tables = torch.zeros((max(G, 1), S, W), dtype=torch.int32, device=self.device)
        return self._records, self._slot_tables

    def _capture_decode_graph(self, b: int):
        layout, words = self._graph_layout(b)
        W, G, S = self.cache.max_pages_per_request, self.num_groups, self.config.max_decode_slots
        records, slot_tables = self._slot_records()
        dev = torch.zeros(words, dtype=torch.int32, device=self.device)
        view = lambda name: dev[layout[name][0]:layout[name][0] + layout[name][1]]
        ctx = StepContext(self)
        ctx.num_tokens = ctx.num_requests = b
        ctx.max_q_len, ctx.decode_only = 1, True
        ctx.max_kv_len = self.config.max_seq_len
        ctx.tokens, ctx.positions, ctx.token_req = view("tok"), view("pos"), view("req")
        ctx.req_indptr, ctx.kv_before, ctx.slots = view("ind"), view("kvb"), view("slot")
        ctx.logit_rows = view("row")
        ctx.num_sampled = b
        ctx.sample_seed = view("seed").view(torch.int64)
        ctx.sample_temperature = view("temp").view(torch.float32)
        ctx.sample_counter = view("count")
        ctx.req_indptr_host = np.arange(b + 1, dtype=np.int32)
        ctx.kv_before_host = np.zeros(b, dtype=np.int32)
        ctx.slots_host = np.zeros(b, dtype=np.int32)
        tables = [dev[o:o + size].view(b, W) for o, size in layout["tables"]]
        lane_tables = dev[layout["tables"][0][0]:] if G else None
        caches = self.storage.layer_caches(tables)
        # the words that never change, and a command block of padding lanes for warm-up and capture
        host = np.zeros(words, dtype=np.int32)
        host[layout["req"][0]:layout["req"][0] + b] = np.arange(b)
        host[layout["ind"][0]:layout["ind"][0] + b + 1] = np.arange(b + 1)
        host[layout["row"][0]:layout["row"][0] + b] = np.arange(b)
        host[2:2 + b] = -1
        dev.copy_(torch.from_numpy(host))
        command = view("command")
        logits = torch.empty((b, self.vocab_size), dtype=torch.float32, device=self.device)
        tokens = torch.empty(b, dtype=torch.int32, device=self.device)

        def body():
            ops.slot_gather(command, b, G, S, W, self.cache.page_size, records, slot_tables, ctx.tokens, ctx.positions,
                            ctx.kv_before, ctx.slots, ctx.sample_seed, ctx.sample_temperature, ctx.sample_counter,
                            lane_tables)
            acc = self.model.forward(ctx, caches)
            self.model.logits(ctx, acc, ctx.logit_rows, logits)
            ops.sample(logits, tokens, ctx.sample_temperature, ctx.sample_seed, ctx.sample_counter)
            ops.slot_advance(command, b, S, tokens, records)

        with torch.no_grad():
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                body()  # warm-up: builds kernels, sizes every scratch buffer
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            launched = ops.launch_count
            with torch.cuda.graph(graph):
                body()
            launched = ops.launch_count - launched
        state = {"kernels": launched, "layout": layout, "words": layout["command"][1], "dev": dev, "graph": graph,
                 "logits": logits, "tokens": tokens}
        self._graphs[b] = state
        return state

    def can_feed_previous(self, entries) -> bool:
        """Whether ``run(entries, feed_previous=True)`` applies: see ``run``."""
        return (self._last_graph_ids is not None and self._graphable(entries)
                and [e.request_id for e in entries] == self._last_graph_ids)

    def tokens_to_host(self, result: StepResult):
        """Starts the copy of a step's sampled tokens into pinned host memory; returns
        (pinned int32 tensor, event).  After ``event.synchronize()`` the tensor holds them.
        Two buffers take turns, so the tokens of two steps can be under way."""
        turn = self._tokens_turn = self._tokens_turn ^ 1
        count = result.tokens.numel()
        if self._tokens_host[turn] is None or self._tokens_host[turn].numel() < count:
            self._tokens_host[turn] = torch.empty(max(count, 256), dtype=torch.int32, pin_memory=True)
            self._tokens_event[turn] = torch.cuda.Event()
        host = self._tokens_host[turn][:count]
        host.copy_(result.tokens, non_blocking=True)
        self._tokens_event[turn].record()
        return host, self._tokens_event[turn]

    def _run_decode_graph(self, entries, feed_previous: bool = False) -> StepResult:
        cache = self.cache
        n = len(entries)
        b = self._bucket(n)
        state = self._graphs.get(b) or self._capture_decode_graph(b)
        layout, words = state["layout"], state["words"]
        W, S = cache.max_pages_per_request, self.config.max_decode_slots
        ids = [e.request_id for e in entries]
        if len(set(ids)) != n:
            raise ValueError("a request appears twice in one step")
        if not feed_previous:
            toks = np.fromiter((e.tokens[0] for e in entries), dtype=np.int32, count=n)
            if n and (toks.min() < 0 or toks.max() >= self.vocab_size):
                raise ValueError(f"token ids must lie in [0, {self.vocab_size})")
        room = cache.begin_decode(ids)
        if not isinstance(room, tuple):
            raise OutOfPages(f"no pages left for request {ids[room]!r}")
        before, slots = room
        # which lanes' slots the device holds no current record (and tables) of
        synced, wants, stale = self._synced, [], []
        for i, e in enumerate(entries):
            want = (e.request_id, int(before[i]), e.sample.counter, float(e.sample.temperature),
                    e.sample.seed & 0x7FFFFFFFFFFFFFFF)
            wants.append(want)
            if synced.get(int(slots[i])) != want:
                stale.append(i)
        page_size, G = cache.page_size, self.num_groups
        stale_words = sum(int(before[i]) // page_size + 1 for i in stale) * G
        # The command block: which slot stands in which lane, and what the device does not know yet.
        host, _ = self._meta(words + stale_words)
        command = host[:words]
        command[:] = 0
        command[0] = n
        lanes, flags = command[2:2 + b], command[2 + b:2 + 2 * b]
        given = command[2 + 2 * b:2 + 8 * b].reshape(6, b)
        pairs = command[2 + 8 * b:]
        lanes[:] = -1
        lanes[:n] = slots
        for i in stale:
            _, position, counter, temperature, seed = wants[i]
            low = seed & 0xFFFFFFFF
            flags[i] = 1
            given[1, i], given[2, i] = position, counter
            given[3, i] = int(np.float32(temperature).view(np.int32))
            given[4, i], given[5, i] = low - (1 << 32) if low >= 1 << 31 else low, seed >> 32
        for i, want in enumerate(wants):  # as the step will leave the records
            synced[int(slots[i])] = (want[0], want[1] + 1, want[2] + 1, want[3], want[4])
        if not feed_previous:
            flags[:n] |= 2
            given[0, :n] = toks
        bytes_sent = words * 4
        records, slot_tables = self._slot_records()
        turn = self._meta_turn
        device_pages = self._device_pages
        if stale:  # a slot that is new to the decode set: its whole table rows, by plain copies
            pinned = self._meta_host[turn]
            room_at = words
            for i in stale:
                slot, used = int(slots[i]), int(before[i]) // page_size + 1
                for g in range(G):
                    host[room_at:room_at + used] = cache.table_arrays[g][slot, :used]
                    slot_tables[g, slot, :used].copy_(pinned[room_at:room_at + used], non_blocking=True)
                    room_at += used
                device_pages[slot] = used
            bytes_sent += stale_words * 4
        # table entries the lanes' slots have gained since their last step (a new page at most)
        count = 0
        used_now = before // page_size + 1
        for i in np.nonzero(used_now > device_pages[slots])[0]:
            slot = int(slots[i])
            for index in range(int(device_pages[slot]), int(used_now[i])):
                for g in range(G):
                    if count >= layout["capacity"]:
                        raise ValueError("more new table entries than a decode step can take")
                    pairs[2 * count] = (g * S + slot) * W + index
                    pairs[2 * count + 1] = cache.table_arrays[g][slot, index]
                    count += 1
        device_pages[slots] = used_now
        command[1] = count
        o = layout["command"][0]
        state["dev"][o:o + words].copy_(self._meta_host[turn][:words], non_blocking=True)
        if self._meta_event[turn] is None:
            self._meta_event[turn] = torch.cuda.Event()
        self._meta_event[turn].record()
        state["graph"].replay()
        ops.launch_count += state["kernels"]
        cache.end_decode(ids)
        self._last_graph_ids = ids
        self.steps_run += 1
        self.graph_steps += 1
        self.h2d_bytes_last_step = bytes_sent
        return StepResult(state["logits"][:n], state["tokens"][:n])

    def _build(self, entries):
        cache = self.cache
        n = len(entries)
        lens = [len(e.tokens) for e in entries]
        T = sum(lens)
        if T > self.token_capacity:
            raise ValueError(f"a step of {T} tokens exceeds the token budget {self.token_capacity}")
        kv_before = [cache.num_tokens(e.request_id) for e in entries]
        seen = set()
        for e, before, q in zip(entries, kv_before, lens):
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if not cache.extend(e.request_id, before + q):
                raise OutOfPages(f"no pages left for request {e.request_id!r} ({before} + {q} tokens)")
        want_rows = []
        offset = 0
        for e, q in zip(entries, lens):
            for w in e.want:
                if not 0 <= w < q:
                    raise ValueError(f"wanted place {w} is outside the {q} tokens of request {e.request_id!r}")
                want_rows.append(offset + w)
            offset += q
        sampled = []
        offset = 0
        for e, q in zip(entries, lens):
            if e.sample is not None:
                sampled.append(e.sample)
                want_rows.append(offset + q - 1)
            offset += q
        k = len(sampled)
        hot = any(s.temperature > 0 for s in sampled)
        m = len(want_rows)
        width = max(1, max(-(-(b + q) // cache.page_size) for b, q in zip(kv_before, lens)))
        G = self.num_groups
        words = 3 * T + (n + 1) + 2 * n + m + G * n * width + (4 * k + 2 if hot else 0)
        host, dev = self._meta(words + T + 4 * n + 1024)  # room for what parts plan on the host
        self._aux_offset = words
        o = 0

        def take(count):
            nonlocal o
            view = (host[o:o + count], dev[o:o + count])
            o += count
            return view

        tok_h, tok_d = take(T)
        pos_h, pos_d = take(T)
        req_h, req_d = take(T)
        ind_h, ind_d = take(n + 1)
        kvb_h, kvb_d = take(n)
        slot_h, slot_d = take(n)
        row_h, row_d = take(m)
        tables = [take(n * width) for _ in range(G)]

        ind_h[0] = 0
        np.cumsum(lens, out=ind_h[1:])
        kvb_h[:] = kv_before
        start = 0
        vocab = self.vocab_size
        for i, (e, before, q) in enumerate(zip(entries, kv_before, lens)):
            tok_h[start:start + q] = e.tokens
            pos_h[start:start + q] = np.arange(before, before + q, dtype=np.int32)
            req_h[start:start + q] = i
            slot_h[i] = cache.slot_of(e.request_id)
            start += q
        slot_index = slot_h[:n]
        for g in range(G):
            np.take(cache.table_arrays[g][:, :width], slot_index, axis=0, out=tables[g][0].reshape(n, width))
        if T and (tok_h[:T].min() < 0 or tok_h[:T].max() >= vocab):
            raise ValueError(f"token ids must lie in [0, {vocab})")
        row_h[:] = want_rows
        if hot:
            o += o & 1  # the 64-bit seeds start on an 8-byte boundary
            seed_h, seed_d = take(2 * k)
            temp_h, temp_d = take(k)
            count_h, count_d = take(k)
            seed_h.view(np.int64)[:] = [s.seed & 0x7FFFFFFFFFFFFFFF for s in sampled]
            temp_h.view(np.float32)[:] = [s.temperature for s in sampled]
            count_h[:] = [s.counter for s in sampled]
        self._upload_meta(words)

        ctx = StepContext(self)
        ctx.num_tokens, ctx.num_requests = T, n
        ctx.max_q_len = max(lens)
        ctx.max_kv_len = max(b + q for b, q in zip(kv_before, lens))
        ctx.decode_only = ctx.max_q_len == 1
        ctx.tokens, ctx.positions, ctx.token_req = tok_d, pos_d, req_d
        ctx.req_indptr, ctx.kv_before, ctx.slots = ind_d, kvb_d, slot_d
        ctx.logit_rows = row_d if m else None
        ctx.num_sampled = k
        ctx.sample_temperature = temp_d.view(torch.float32) if hot else None
        ctx.sample_seed = seed_d.view(torch.int64) if hot else None
        ctx.sample_counter = count_d if hot else None
        ctx.req_indptr_host, ctx.kv_before_host, ctx.slots_host = ind_h.copy(), kvb_h.copy(), slot_h.copy()
        block_tables = [t[1].view(n, width) for t in tables]
        return ctx, self.storage.layer_caches(block_tables)
