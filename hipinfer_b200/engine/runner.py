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
                 max_num_seqs: int = 8):
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

    # ---------------------------------------------------------------- construction helpers
    @classmethod
    def from_folder(cls, folder: str, **kw) -> "ModelRunner":
        config = load_config(folder)
        spec = get_architecture(config.architecture).build_spec(config)
        from ..parts.spec import spec_param_specs

        tensors = load_weights(folder, spec_param_specs(spec), device=kw.get("device", "cuda:0"),
                               ignore=_ignorable(spec))
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

    def check_entries(self, entries: Sequence[StepEntry]) -> None:
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            if n < 1:
                raise StepError(f"request {e.request_id!r}: an entry needs at least one token")
            for t in e.tokens:
                if not (0 <= int(t) < self.vocab_size):
                    raise StepError(f"request {e.request_id!r}: token {t} is outside the vocabulary of "
                                    f"{self.vocab_size}")
            if self.length(e.request_id) + n > self.max_model_len:
                raise StepError(f"request {e.request_id!r}: {self.length(e.request_id)} + {n} tokens exceed the "
                                f"longest sequence of {self.max_model_len}")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"request {e.request_id!r}: want {w} is outside its {n} tokens")

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one batch; float32 logits [number of wanted places, vocab] on the device.
        Raises OutOfPages (nothing changed) when the cache cannot hold the new tokens."""
        entries = list(entries)
        self.check_entries(entries)
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
            rc = self.cache.get(e.request_id)
            ctx_lens.append(rc.length)
            slots.append(rc.state_slot)
            slot_maps.append(self.cache.append(e.request_id, len(e.tokens)))
            tables.append([list(t) for t in rc.tables])
        batch = build_step_batch(entries, ctx_lens, slots, tables, slot_maps, len(self.cache.groups), self.device)
        logits = self.model.forward(batch, self.storage)
        for e in entries:
            self.cache.release_behind_window(e.request_id)
        self.steps_run += 1
        return logits

    def end(self, request_id) -> None:
        """The request is finished: its pages and its state slot are given back."""
        self.cache.free_request(request_id)

    def live_requests(self):
        return list(self.cache.requests)


def _ignorable(spec) -> List[str]:
    """Tensors a checkpoint may carry that the model does not read: a stored copy of the head
    of a model whose head is tied to the embedding is NOT among them (it would be silently
    dropped); rotary inv_freq buffers of older files are."""
    return [f"{ls.prefix}self_attn.rotary_emb.inv_freq" for ls in spec.layers]
