"""The Python entry point, in the manner of the reference's binding (scripts/hipinfer.py:334-516):

    eng = Engine(path, max_batch=8, max_seq=2048, max_prefill=1024)
    tokens = eng.generate(prompt_ids, n_new)            # greedy; n_new tokens, the first from the prompt
    eng.close()

with the same attribute names (`vocab, hidden, inter, layers, heads, kv_heads, head_dim,
max_pos, tied, weight_bytes, kv_bytes_per_token`), the slot calls `prefill(slot, tokens, p0)`,
`prefill_logits`, `decode(B, steps)`, `history(slot, start, n)`, `logits(B)`, and `ValueError`
for bad arguments (scripts/hipinfer.py:386-390). What is new beside them: `dtype`
("bfloat16" or "float32"), temperature sampling, requests through the scheduler
(`add_request`, `step`, `run`), random weights, and `runner` for the step function itself.

`max_batch` is the most requests live at a time, `max_seq` the longest sequence, `max_prefill`
the token budget of a step (the reference's prefill chunk, src/api.cu:1788).
"""
from __future__ import annotations

import itertools
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..cache import OutOfPages
from ..config import ModelConfig, config_from_dict, load_config
from ..kernels import ops
from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .runner import ModelRunner, StepError
from .scheduler import AdmissionError, Request, Scheduler


class Engine:
    def __init__(self, path: Optional[str] = None, max_batch: int = 8, max_seq: int = 2048, max_prefill: int = 1024,
                 dtype: str = "bfloat16", device: str = "cuda:0", config: Union[ModelConfig, dict, None] = None,
                 random_weights: Optional[int] = None, std: float = 0.02, page_size: int = 16,
                 num_pages: Optional[int] = None, pipeline: bool = True):
        kw = dict(dtype=dtype, device=device, page_size=page_size, num_pages=num_pages, max_model_len=max_seq,
                  max_num_seqs=max_batch)
        if path is not None:
            self.runner = ModelRunner.from_folder(path, **kw)
        elif config is not None and random_weights is not None:
            cfg = config_from_dict(config) if isinstance(config, dict) else config
            self.runner = ModelRunner.from_random(cfg, seed=random_weights, std=std, **kw)
        else:
            raise ValueError("Engine needs a model folder, or config= and random_weights=seed")
        r = self.runner
        self.max_batch, self.max_seq, self.max_prefill = max_batch, r.max_model_len, max_prefill
        self.device, self.dtype = r.device, dtype
        self.scheduler = Scheduler(r.cache, max_batch, max_prefill, r.max_model_len, r.spec.eos_token_ids)
        self.sampler = Sampler(r.device)
        c = r.config
        self.vocab = r.spec.vocab_size
        self.hidden = r.spec.hidden_size
        self.max_pos = r.spec.max_position
        for ours, theirs in (("inter", "intermediate_size"), ("layers", "num_hidden_layers"),
                             ("heads", "num_attention_heads"), ("kv_heads", "num_key_value_heads"),
                             ("head_dim", "head_dim"), ("tied", "tie_word_embeddings")):
            setattr(self, ours, getattr(c, theirs, None))
        self.weight_bytes = r.model.step_weight_bytes()
        self.kv_bytes_per_token = r.storage.bytes_per_token()
        # pipeline: a step is launched before the tokens of the step before it have been read
        # back, so the host prepares step i + 1 while the device runs step i (see step())
        self.pipeline = bool(pipeline)
        self._pending = None
        self._copy_stream = torch.cuda.Stream(device=r.device)
        self.last_step = None      # (rows, requests, rows of prompt portions) of the step launched last
        self._unreported: List[Request] = []
        self._ids = itertools.count()
        self._slots: Dict[int, dict] = {}
        self._last_logits: Dict[int, torch.Tensor] = {}

    # ---------------------------------------------------------------- requests through the scheduler
    def add_request(self, prompt: Sequence[int], n_new: int, temperature: float = 0.0, seed: int = 0,
                    stop_token_ids: Sequence[int] = (), ignore_eos: bool = True, request_id=None):
        for t in prompt:
            if not (0 <= int(t) < self.vocab):
                raise ValueError(f"token {t} is outside the vocabulary of {self.vocab}")
        rid = next(self._ids) if request_id is None else request_id
        params = SamplingParams(temperature, seed, n_new, tuple(stop_token_ids), ignore_eos)
        try:
            self.scheduler.add(Request(rid, [int(t) for t in prompt], params))
        except AdmissionError as e:
            raise ValueError(str(e)) from None
        return rid

    def step(self) -> List[Request]:
        """One scheduler step: schedule, run the batch, sample, record. Returns requests whose
        last token has arrived on the host.

        With `pipeline` the sampled tokens stay on the device and feed the next step there; the
        step is recorded with placeholders, the NEXT step is scheduled and launched, and only then
        are this step's tokens read back. The host's work for a step thus overlaps the device's
        work for the step before. Finishing by length needs no token value; a stop token is
        noticed one step late, and the extra token is dropped."""
        if not self.pipeline:
            return self._step_sync()
        done: List[Request] = []
        sched = self.scheduler.schedule() if self.scheduler.has_work() else []
        if not sched:
            if self.scheduler.has_work() and self._pending is None:
                raise RuntimeError("the scheduler has work but could schedule nothing")
            return self._collect()
        if self._pending is not None and any(self._inner_placeholder(s) for s in sched):
            done += self._collect()            # a portion needs a token value that is still on the device
        older = self._pending
        self._pending = self._launch(sched, older)
        if older is not None:
            done += self._collect(older)
        return done

    PLACEHOLDER = -1

    def _inner_placeholder(self, s) -> bool:
        toks = s.request.tokens
        part = toks[s.start:s.start + s.n]
        if self.PLACEHOLDER not in part:
            return False
        return part.count(self.PLACEHOLDER) > 1 or part[-1] != self.PLACEHOLDER or s.start + s.n != len(toks)

    def _launch(self, sched, older):
        """Run the batch and sample on the device; record the step with placeholders."""
        entries, token_map, row = [], [], 0
        src = {id(req): i for i, (req, _) in enumerate(older["slots"])} if older is not None else {}
        for s in sched:
            part = list(s.request.tokens[s.start:s.start + s.n])
            tm = [-1] * s.n
            if part[-1] == self.PLACEHOLDER:
                part[-1] = 0
                tm[-1] = src[id(s.request)]
            entries.append(StepEntry(s.request.request_id, part, [s.n - 1] if s.samples else []))
            token_map += tm
            row += s.n
        self.last_step = (row, len(sched), sum(s.n for s in sched if s.n > 1))
        feed = older is not None and any(t >= 0 for t in token_map)
        logits = self.runner.step(entries, device_tokens=older["tokens_dev"] if feed else None,
                                  token_map=token_map if feed else None)
        samplers = [s for s in sched if s.samples]
        pending = dict(slots=[], tokens_dev=None, host=None, event=None)
        if samplers:
            tokens_dev = self.sampler.sample_device(logits, [s.request.params for s in samplers],
                                                    [s.start + s.n for s in samplers])
            # the tokens go to the host on a stream of their own: a copy in the compute stream would stand between this
            # step's last kernel and the next step's first (the copy engine's turn-around, some 10 us a step)
            host = torch.empty(len(samplers), dtype=torch.int32, pin_memory=True)
            sampled = torch.cuda.Event()
            sampled.record()
            event = torch.cuda.Event()
            with torch.cuda.stream(self._copy_stream):
                self._copy_stream.wait_event(sampled)
                host.copy_(tokens_dev, non_blocking=True)
                event.record(self._copy_stream)
            tokens_dev.record_stream(self._copy_stream)
            pending.update(tokens_dev=tokens_dev, host=host, event=event)
        self.scheduler.update(sched, [self.PLACEHOLDER] * len(samplers))
        pending["slots"] = [(s.request, len(s.request.output) - 1) for s in samplers]
        self._unreported += [s.request for s in samplers if s.request.status == "finished"]
        return pending

    def _collect(self, pending=None) -> List[Request]:
        """Read a launched step's tokens, put them in the place of their placeholders, apply the
        stop conditions that need a token's value, and report requests that are complete."""
        if pending is None:
            pending, self._pending = self._pending, None
        if pending is not None and pending["event"] is not None:
            pending["event"].synchronize()
            ops.check_device_status()          # raises KernelTimeout if a kernel of the step gave up on a wait
            eos = self.scheduler.eos
            for (req, idx), tok in zip(pending["slots"], pending["host"].tolist()):
                if idx >= len(req.output):
                    continue                   # cut off by a stop token found earlier
                req.output[idx] = tok
                p = req.params
                if tok in p.stop_token_ids or (not p.ignore_eos and tok in eos):
                    del req.output[idx + 1:]
                    if req.status != "finished":
                        self.scheduler.finish(req, "stop")
                        self._unreported.append(req)
                    else:
                        req.finish_reason = "stop"
        done = [r for r in self._unreported if self.PLACEHOLDER not in r.output]
        self._unreported = [r for r in self._unreported if self.PLACEHOLDER in r.output]
        return done

    def _step_sync(self) -> List[Request]:
        sched = self.scheduler.schedule()
        if not sched:
            if self.scheduler.has_work():
                raise RuntimeError("the scheduler has work but could schedule nothing")
            return []
        entries = [StepEntry(s.request.request_id, s.request.tokens[s.start:s.start + s.n], [s.n - 1] if s.samples else [])
                   for s in sched]
        self.last_step = (sum(s.n for s in sched), len(sched), sum(s.n for s in sched if s.n > 1))
        logits = self.runner.step(entries)
        samplers = [s for s in sched if s.samples]
        toks = self.sampler.sample(logits, [s.request.params for s in samplers],
                                   [s.start + s.n for s in samplers])
        return self.scheduler.update(sched, toks)

    def run(self) -> Dict[object, List[int]]:
        """Step until every added request has finished; {request id: produced tokens}."""
        out = {}
        while self.scheduler.has_work() or self._pending is not None or self._unreported:
            for req in self.step():
                out[req.request_id] = list(req.output)
        return out

    def abort_all(self) -> None:
        """Drop every request: wait for a step in flight, then free all pages and state slots."""
        self._collect()
        self._unreported = []
        for req in list(self.scheduler.running) + list(self.scheduler.waiting):
            self.scheduler.finish(req, "aborted")
        self.scheduler.waiting.clear()

    def generate(self, prompt, n_new: int, graph: bool = True, temperature: float = 0.0, seed: int = 0):
        """n_new tokens after `prompt` (the first comes from the prompt's last position).
        A list of prompts gives a list of results; they run as one batch."""
        many = bool(prompt) and isinstance(prompt[0], (list, tuple))
        prompts = list(prompt) if many else [prompt]
        ids = [self.add_request(p, n_new, temperature, seed) for p in prompts]
        res = self.run()
        outs = [res[i] for i in ids]
        return outs if many else outs[0]

    # ---------------------------------------------------------------- the reference's slot calls
    def _slot_ok(self, slot):
        if not (0 <= slot < self.max_batch):
            raise ValueError(f"slot {slot} is outside [0, {self.max_batch})")

    def _run_tokens(self, slot: int, tokens: Sequence[int], p0: int, all_logits: bool):
        self._slot_ok(slot)
        rid = ("slot", slot)
        tokens = [int(t) for t in tokens]
        if not tokens:
            raise ValueError("prefill needs at least one token")
        if p0 < 0 or p0 + len(tokens) > self.max_seq:
            raise ValueError(f"positions [{p0}, {p0 + len(tokens)}) exceed the longest sequence {self.max_seq}")
        if any(not (0 <= t < self.vocab) for t in tokens):
            raise ValueError(f"a token is outside the vocabulary of {self.vocab}")
        st = self._slots.get(slot)
        held = len(st["tokens"]) if st else 0
        if p0 != 0 and p0 != held:
            raise ValueError(f"slot {slot} holds {held} tokens; cannot continue at p0={p0}")
        if p0 == 0:                                   # a fresh start of the slot
            if self.runner.cache.has_request(rid):
                self.runner.end(rid)
            st = self._slots[slot] = dict(tokens=[])
        rows = []
        try:
            for t0 in range(0, len(tokens), self.max_prefill):
                part = tokens[t0:t0 + self.max_prefill]
                last = t0 + len(part) == len(tokens)
                want = list(range(len(part))) if all_logits else ([len(part) - 1] if last else [])
                lg = self.runner.step([StepEntry(rid, part, want)])
                if lg.shape[0]:
                    rows.append(lg)
        except (StepError, OutOfPages) as e:
            raise ValueError(str(e)) from None
        st["tokens"].extend(tokens)
        logits = torch.cat(rows) if len(rows) > 1 else rows[0]
        self._last_logits[slot] = logits[-1]
        return logits

    def prefill(self, slot: int, tokens: Sequence[int], p0: int = 0) -> int:
        """Run `tokens` at positions p0.. of `slot`; returns the first new token (greedy) and
        keeps it as the slot's next input (src/api.cu:1771-1822)."""
        logits = self._run_tokens(slot, tokens, p0, False)
        tok = self.sampler.sample(logits[-1:], [SamplingParams()], [0])[0]
        self._slots[slot]["next"] = tok
        return tok

    def prefill_logits(self, slot: int, tokens: Sequence[int], p0: int = 0) -> torch.Tensor:
        """Prefill and return the float32 logits of every position, [T, vocab] on the GPU."""
        return self._run_tokens(slot, tokens, p0, True)

    def decode(self, B: int, steps: int, graph: bool = True) -> float:
        """`steps` greedy tokens for slots [0, B), each from its own position; returns GPU milliseconds."""
        if not (1 <= B <= self.max_batch) or any(s not in self._slots or "next" not in self._slots[s] for s in range(B)):
            raise ValueError(f"decode needs slots [0, {B}) prefilled")
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        try:
            for _ in range(steps):
                entries = [StepEntry(("slot", s), [self._slots[s]["next"]], [0]) for s in range(B)]
                logits = self.runner.step(entries)
                toks = self.sampler.sample(logits, [SamplingParams()] * B, [0] * B)
                for s in range(B):
                    self._slots[s]["tokens"].append(self._slots[s]["next"])
                    self._slots[s]["next"] = toks[s]
                    self._last_logits[s] = logits[s]
        except (StepError, OutOfPages) as e:
            raise ValueError(str(e)) from None
        stop.record()
        stop.synchronize()
        ops.check_device_status()
        return start.elapsed_time(stop)

    def history(self, slot: int, start: int, n: int) -> List[int]:
        """Tokens of `slot` at positions [start, start + n): the prompt, then what was generated."""
        self._slot_ok(slot)
        st = self._slots.get(slot)
        seq = (st["tokens"] + [st["next"]]) if st and "next" in st else (st["tokens"] if st else [])
        if start < 0 or n < 0 or start + n > len(seq):
            raise ValueError(f"slot {slot} holds positions [0, {len(seq)}); asked for [{start}, {start + n})")
        return seq[start:start + n]

    def logits(self, B: int) -> torch.Tensor:
        """The last logits of slots [0, B), float32 [B, vocab] on the GPU."""
        if any(s not in self._last_logits for s in range(B)):
            raise ValueError(f"logits needs slots [0, {B}) run")
        return torch.stack([self._last_logits[s] for s in range(B)])

    def close(self):
        self.runner = None
        self.scheduler = None
        self._slots.clear()
        self._last_logits.clear()
        torch.cuda.empty_cache()
