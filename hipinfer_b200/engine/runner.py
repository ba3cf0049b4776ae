"""The step function. `ModelRunner.step(entries)` takes a batch of (request, its next tokens):
portions of prompts beside single decoded tokens, cut anywhere. It makes room in the cache,
runs only the tokens it is given, as one batch, from the cache earlier steps left, and returns
the 32-bit logits at the wanted places, in the order of the entries and of their `want`.
Generation, the scheduler and trace replay all go through this one function.

A request is known from the first step that names it until `end(request_id)`; its position is
the number of tokens it has been given so far.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, CacheStorage, OutOfPages
from ..config import ModelConfig, get_architecture, load_config
from ..models.decoder import DecoderModel
from ..parts.registry import BuildContext
from ..weights import load_weights, random_weights
from .batch import StepBatch, StepEntry, build_step_batch

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class StepError(ValueError):
    """A step that cannot run: a token outside the vocabulary, a request beyond the longest
    sequence, a `want` outside the entry (the reference returns -1 for such arguments,
    src/api.cu:1827-1839)."""


class ModelRunner:
    def __init__(self, config: ModelConfig, tensors: Dict[str, torch.Tensor], dtype="bfloat16", device="cuda:0",
                 page_size: int = 16, num_pages: Optional[int] = None, max_model_len: Optional[int] = None,
                 max_num_seqs: int = 8, cuda_graphs: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("hipinfer_b200 runs on a CUDA device (sm_100a); none is visible and there is no "
                               "CPU implementation")
        self.config = config
        self.dtype = DTYPES[dtype] if isinstance(dtype, str) else dtype
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.spec = get_architecture(config.architecture).build_spec(config)
        self.max_model_len = int(min(max_model_len or self.spec.max_position, self.spec.max_position))
        self.page_size = int(page_size)
        self.ctx = BuildContext(self.dtype, self.device, self.page_size, self.max_model_len)
        self.model = DecoderModel(self.spec, self.ctx)
        self.model.load(tensors)
        pages_per_seq = -(-self.max_model_len // self.page_size)
        n_pages = int(num_pages) if num_pages is not None else pages_per_seq * max_num_seqs
        groups = self.model.cache_groups
        self.cache = CacheManager(groups, self.page_size, [n_pages] * len(groups), max_num_seqs)
        self.storage = CacheStorage(groups, [n_pages] * len(groups), self.page_size, self.dtype, self.device,
                                    self.model.state_specs, max_num_seqs)
        self.vocab_size = self.spec.vocab_size
        self.steps_run = 0
        # decode-only steps (one token per request, every row wanted) are replayed from a CUDA
        # graph captured per number of requests: same kernels, one launch
        self.cuda_graphs = bool(cuda_graphs)
        self._graphs: Dict[tuple, dict] = {}
        self._graph_pool = None
        self._table_widths = [pages_per_seq] * len(groups)
        self._np_tables: Dict[object, list] = {}

    # ---------------------------------------------------------------- construction helpers
    @classmethod
    def from_folder(cls, folder: str, **kw) -> "ModelRunner":
        config = load_config(folder)
        spec = get_architecture(config.architecture).build_spec(config)
        from ..parts.spec import spec_param_specs

        dt = kw.get("dtype", "bfloat16")
        exact = (DTYPES[dt] if isinstance(dt, str) else dt) == torch.float32
        tensors = load_weights(folder, spec_param_specs(spec), device=kw.get("device", "cuda:0"),
                               ignore=_ignorable(spec), half_as=torch.float32 if exact else torch.bfloat16)
        return cls(config, tensors, **kw)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int = 0, std: float = 0.02, norm_std: float = 0.0,
                    weights_dtype=torch.bfloat16, **kw) -> "ModelRunner":
        from ..parts.spec import spec_param_specs

        spec = get_architecture(config.architecture).build_spec(config)
        tensors = random_weights(spec_param_specs(spec), seed, std, norm_std, weights_dtype,
                                 device=kw.get("device", "cuda:0"))
        return cls(config, tensors, **kw)

    # ---------------------------------------------------------------- the step
    def length(self, request_id) -> int:
        return self.cache.get(request_id).length if self.cache.has_request(request_id) else 0

    def check_entries(self, entries: Sequence[StepEntry]) -> list:
        """Raises StepError for a batch that cannot run; returns the entries' tokens as int64 arrays."""
        seen, arrays = set(), []
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            if n < 1:
                raise StepError(f"request {e.request_id!r}: an entry needs at least one token")
            toks = np.asarray(e.tokens, dtype=np.int64)          # one pass, not a Python loop: a portion may have thousands
            if toks.ndim != 1:
                raise StepError(f"request {e.request_id!r}: tokens must be a flat sequence of ints")
            bad = (toks < 0) | (toks >= self.vocab_size)
            if bad.any():
                raise StepError(f"request {e.request_id!r}: token {int(toks[bad][0])} is outside the vocabulary of "
                                f"{self.vocab_size}")
            if self.length(e.request_id) + n > self.max_model_len:
                raise StepError(f"request {e.request_id!r}: {self.length(e.request_id)} + {n} tokens exceed the "
                                f"longest sequence of {self.max_model_len}")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"request {e.request_id!r}: want {w} is outside its {n} tokens")
            arrays.append(toks)
        return arrays

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None,
             token_map: Optional[Sequence[int]] = None, dump: Optional[dict] = None) -> torch.Tensor:
        """Run one batch; float32 logits [number of wanted places, vocab] on the device.
        Raises OutOfPages (nothing changed) when the cache cannot hold the new tokens.
        `device_tokens` (int32 [rows], on the device) replaces the entries' token values, which
        are then placeholders: tokens sampled on the device feed the next step without a trip to
        the host (the reference keeps token and position on the device for the same reason,
        README.md:510-512). With `token_map` (one int per row) only rows with an entry >= 0 take
        their token from device_tokens[entry]; the others keep the value the entry gives.
        `dump` (a dict): the step runs eagerly and leaves named planes of every layer in it (parts/planes.py)."""
        entries = list(entries)
        token_arrays = self.check_entries(entries)
        if not entries:
            return torch.empty(0, self.vocab_size, dtype=torch.float32, device=self.device)
        # room for everything first, so that a failure leaves no request half advanced
        new = [e.request_id for e in entries if not self.cache.has_request(e.request_id)]
        need = [0] * len(self.cache.groups)
        for e in entries:
            for g, n in enumerate(self.cache.pages_needed(e.request_id, len(e.tokens))):
                need[g] += n
        for g, n in enumerate(need):
            if n > self.cache.pools[g].free_count:
                raise OutOfPages(f"cache group {self.cache.groups[g].name!r}: this step needs {n} more pages, "
                                 f"{self.cache.pools[g].free_count} are free")
        if len(new) > self.cache.slots.free_count:
            from ..cache import OutOfStateSlots
            raise OutOfStateSlots(f"{len(new)} new requests, {self.cache.slots.free_count} state slots free")
        ctx_lens, slots, tables, slot_maps = [], [], [], []
        for e in entries:
            if not self.cache.has_request(e.request_id):
                rc = self.cache.add_request(e.request_id)
                self.storage.zero_state_slot(rc.state_slot)
                self._np_tables.pop(e.request_id, None)    # an id that comes back (after preemption) starts afresh
            rc = self.cache.get(e.request_id)
            ctx_lens.append(rc.length)
            slots.append(rc.state_slot)
            slot_maps.append(self.cache.append(e.request_id, len(e.tokens), as_arrays=True))
            tables.append(self._table_rows(rc))
        if dump is None and self.cuda_graphs and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            logits = self._graph_step(entries, ctx_lens, slots, tables, slot_maps, device_tokens, token_map)
        else:
            batch = build_step_batch(entries, ctx_lens, slots, tables, slot_maps, len(self.cache.groups), self.device,
                                     token_map=token_map, token_arrays=token_arrays)
            self._feed(batch.tokens, batch.token_map, device_tokens, token_map)
            batch.dump = dump
            logits = self.model.forward(batch, self.storage)
        for e in entries:
            if self.cache.release_behind_window(e.request_id):
                self._np_tables.pop(e.request_id, None)
        if len(self._np_tables) > len(self.cache.requests):      # requests freed through the cache manager (the scheduler does)
            for rid in [r for r in self._np_tables if not self.cache.has_request(r)]:
                del self._np_tables[rid]
        self.steps_run += 1
        return logits

    def _table_rows(self, rc):
        """The request's block tables as int32 arrays, kept between steps and extended by the new pages only."""
        rows = self._np_tables.setdefault(rc.request_id, [[np.full(16, -1, dtype=np.int32), 0] for _ in rc.tables])
        out = []
        for slot, table in zip(rows, rc.tables):
            arr, n = slot
            if len(table) > arr.shape[0]:
                grown = np.full(2 * len(table), -1, dtype=np.int32)
                grown[:n] = arr[:n]
                slot[0] = arr = grown
            if len(table) > n:
                arr[n:len(table)] = table[n:]
                slot[1] = len(table)
            out.append(arr[:len(table)])
        return out

    @staticmethod
    def _feed(tokens, map_dev, device_tokens, token_map):
        if device_tokens is None:
            return
        if token_map is None:
            tokens.copy_(device_tokens, non_blocking=True)
        else:
            from ..kernels import ops
            ops.feed_tokens(tokens, device_tokens, map_dev)

    GRAPH_LENGTH_QUANTUM = 512     # tokens by which the length class of a decode graph grows
    MAX_GRAPHS = 128               # captured graphs kept, least recently used first to go (each holds its batch buffer
                                   # and its logits; what a step allocates besides comes from one pool they share)

    def _graph_step(self, entries, ctx_lens, slots, tables, slot_maps, device_tokens=None, token_map=None) -> torch.Tensor:
        """A decode-only step through the CUDA graph for this many requests and this length class (captured at
        first use). The graph's batch lives in one static device buffer that each step overwrites; launch
        geometry is made for the longest position of the class (the step's longest request rounded up to
        GRAPH_LENGTH_QUANTUM tokens), so few blocks lie beyond a row's keys and those return at once; a new
        graph is captured when the longest request crosses into the next class. The logits tensor is the
        graph's own and is overwritten by the next such step."""
        R, G = len(entries), len(self.cache.groups)
        bound = min(self.max_model_len, (max(ctx_lens) // self.GRAPH_LENGTH_QUANTUM + 1) * self.GRAPH_LENGTH_QUANTUM)
        key = (R, bound)
        g = self._graphs.get(key)
        args = dict(n_groups=G, device=self.device, table_widths=self._table_widths, max_pos=bound - 1)
        if g is None:
            n_int = 4 * R + 4 * R + R + sum(R * w for w in self._table_widths) + G * R
            static = torch.zeros(n_int, dtype=torch.int32, device=self.device)
            batch = build_step_batch(entries, ctx_lens, slots, tables, slot_maps, static=static, token_map=token_map, **args)
            self._feed(batch.tokens, batch.token_map, device_tokens, token_map)
            first = self.model.forward(batch, self.storage)    # this step itself, run eagerly: allocations, plans, lazy set-up
            torch.cuda.synchronize()
            from ..kernels import library
            before = library.launches[0]
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            # one memory pool for all graphs: they never run at the same time, and what a step allocates and frees
            # on its way is the same memory in every graph (only the logits, which stay alive, are a graph's own)
            with torch.cuda.graph(graph, pool=self._graph_pool):     # recorded, not run
                logits = self.model.forward(batch, self.storage)
            while len(self._graphs) >= self.MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = dict(graph=graph, static=static, logits=logits, tokens=batch.tokens,
                                   token_map=batch.token_map, launches=library.launches[0] - before)
            # the step has run once already: replaying the graph now would run it a second time, which a mixer
            # with state of its own (its state advances with every run) must not see
            return first
        else:
            self._graphs[key] = self._graphs.pop(key)          # most recently used last
            build_step_batch(entries, ctx_lens, slots, tables, slot_maps, static=g["static"], token_map=token_map, **args)
            self._feed(g["tokens"], g["token_map"], device_tokens, token_map)
        g["graph"].replay()
        from ..kernels import library
        library.launches[0] += g["launches"]
        return g["logits"]

    def end(self, request_id) -> None:
        """The request is finished: its pages and its state slot are given back."""
        self.cache.free_request(request_id)
        self._np_tables.pop(request_id, None)

    def live_requests(self):
        return list(self.cache.requests)


def _ignorable(spec) -> List[str]:
    """Tensors a checkpoint may carry that the model does not read: a stored copy of the head
    of a model whose head is tied to the embedding is NOT among them (it would be silently
    dropped); rotary inv_freq buffers of older files are."""
    return [f"{ls.prefix}self_attn.rotary_emb.inv_freq" for ls in spec.layers]
