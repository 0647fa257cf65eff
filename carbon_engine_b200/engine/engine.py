"""The Python entry point: load a model folder, generate tokens for prompts.

``Engine`` does what the reference's ``Engine::load`` + ``scheduler::spawn`` + ``submit`` do
together (src/engine.rs:140-404, src/scheduler.rs:385-440, 199-231): read the config, pick the
model from the registry, load the weights (or random ones), size the cache, then run the
scheduler's steps through the step function and the sampler until every request is done.
Argument names follow the reference's engine flags (src/main.rs:103-217).
"""
from __future__ import annotations

import json
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..cache.storage import CacheStorage
from ..config.registry import load_config, resolve_architecture
from ..csrc.kernel_lib import kernels
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, fresh_seed, top_logprobs
from ..weights.loader import load_from_folder, load_random
from .batch import StepEntry
from ..cache.manager import CacheError
from ..csrc.kernel_lib import KernelError
from .runner import ModelRunner, StepError
from .scheduler import PlanEntry, Scheduler, SubmitError

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "f32": torch.float32,
          "auto": torch.bfloat16}


def parse_dtype(name: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name} is not supported (bfloat16 or float32)")
        return name
    try:
        return DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype '{name}' is not supported (auto, bf16/bfloat16, f32/float32)") from None


def require_gpu(device: Union[str, torch.device]) -> torch.device:
    dev = torch.device(device)
    if dev.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("this engine runs on a CUDA device only; there is no CPU path")
    kernels()            # fails loudly here if the kernel library cannot be built or loaded
    torch.cuda.set_device(dev)
    return dev


def build_model(model_dir: Optional[str], dtype: torch.dtype, device: torch.device, *, config=None,
                hf_overrides: Optional[Dict[str, Any]] = None, dummy_weight: bool = False, seed: int = 0,
                max_seq_len: int = 0):
    """(model, config, max_seq_len): the model of a folder (or of a typed config) with weights loaded."""
    if config is None:
        arch, config = load_config(model_dir, hf_overrides)
    else:
        arch = resolve_architecture(config.to_json_dict())
    # the context cap: the flag, else the checkpoint's, capped at 32768 (src/engine.rs:177-181)
    if max_seq_len <= 0:
        max_seq_len = min(config.max_position_embeddings, 32768)
    model = arch.build_model(config, max_seq_len)
    if dummy_weight or model_dir is None:
        load_random(model, seed, device, dtype)
    else:
        load_from_folder(model, model_dir, device, dtype)
    return model, config, max_seq_len


@dataclass
class RequestOutput:
    request_id: int
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: str
    error: Optional[str] = None
    logprobs: Optional[List[dict]] = None

    @property
    def usage(self) -> Dict[str, int]:
        return {"prompt_tokens": len(self.prompt_token_ids), "completion_tokens": len(self.token_ids)}


@dataclass
class _Live:
    params: SamplingParams
    seed: int
    prompt: List[int]
    adopted: bool = False
    logprobs: List[dict] = field(default_factory=list)


@dataclass
class _InFlight:
    """A step that is on the device and whose picks have not been read."""
    ids: List[int]                      # the requests it samples for, in the order of its picks
    starts: Dict[int, int]              # where each request's tokens of this step begin
    steps: List[int] = field(default_factory=list)       # tokens each request had drawn before it
    want_lp: List[int] = field(default_factory=list)
    base: Any = None
    picks: Optional[torch.Tensor] = None
    ticket: Any = None


class Engine:
    def __init__(self, model: Optional[str] = None, *, config=None, dtype: Union[str, torch.dtype] = "auto",
                 device: str = "cuda:0", hf_overrides: Optional[Dict[str, Any]] = None, dummy_weight: bool = False,
                 seed: int = 0, kv_tokens: Optional[int] = None, memory_ratio: float = 0.9, page_size: int = 16,
                 max_seq_len: int = 0, max_running_requests: int = 16, max_prefill_tokens: int = 4096,
                 cuda_graphs: bool = False, poison_cache: bool = False, host_lookahead: bool = True,
                 run_ahead: bool = True):
        self.device = require_gpu(device)
        self.dtype = parse_dtype(dtype)
        self.model, self.config, self.max_seq_len = build_model(
            model, self.dtype, self.device, config=config, hf_overrides=hf_overrides, dummy_weight=dummy_weight,
            seed=seed, max_seq_len=max_seq_len)
        self.page_size = int(page_size)
        self.max_running = int(max_running_requests)
        self.max_step_tokens = max(int(max_prefill_tokens), self.max_running)
        num_pages = self._size_cache(kv_tokens, memory_ratio)
        self.storage = CacheStorage(self.model, self.dtype, self.device, self.page_size, num_pages, self.max_running,
                                    self.max_seq_len, poison=poison_cache)
        self.runner = ModelRunner(self.model, self.storage, self.max_step_tokens)
        self.scheduler = Scheduler(self.storage.manager, self.max_running, self.max_step_tokens, self.max_seq_len,
                                   self.config.vocab_size, self.config.eos_token_ids)
        self.sampler = Sampler(self.device)
        self.cuda_graphs = bool(cuda_graphs) and self.runner.enable_graphs()
        self._live: Dict[int, _Live] = {}
        self._done: Dict[int, RequestOutput] = {}
        self._next_id = 0
        self.d2h_bytes_last = 0
        self._last_error: Optional[str] = None
        #: (request, token, its log-probability entry or None) of every token the last step sampled
        self.last_sampled: List[tuple] = []
        # while a decode step runs, the next one is laid out on the host on the guess that the same requests go on
        self.host_lookahead = bool(host_lookahead)
        # ... and launched too, where that guess can only fail by an end token or an abort (see ``step``)
        self.run_ahead = bool(run_ahead)
        self._in_flight: Optional[_InFlight] = None
        self.run_ahead_steps = 0             # steps launched before the step before them was read

    # -- sizing ---------------------------------------------------------------------------------
    def _bytes_per_token(self) -> int:
        from ..parts.base import PagedCacheSpec
        el = 2 if self.dtype == torch.bfloat16 else 4
        return sum(2 * s.kv_heads * s.head_dim * el for _, s in self.model.cache_layout()
                   if isinstance(s, PagedCacheSpec))

    def _state_bytes(self) -> int:
        """Bytes of the fixed-size per-request state of every slot (src/model/mod.rs:129-145 counts them too)."""
        from ..parts.base import StateCacheSpec
        el = 2 if self.dtype == torch.bfloat16 else 4
        total = 0
        for _, s in self.model.cache_layout():
            if isinstance(s, StateCacheSpec):
                n = 1
                for dim in s.shape:
                    n *= int(dim)
                total += n * (torch.empty((), dtype=s.dtype).element_size() if s.dtype is not None else el)
        return total * self.max_running

    def _workspace_bytes(self) -> int:
        """What has to stay free beside the cache: the activations of the largest step (a quarter more, for the
        allocator's rounding), the split-K and split-KV scratch, and a margin for the CUDA context's own needs."""
        from .. import ops_tensor
        el = 2 if self.dtype == torch.bfloat16 else 4
        step = self.model.step_bytes(self.max_step_tokens, el, rows=self.max_running)
        return step + step // 4 + 4 * ops_tensor.GEMM_SCRATCH_FLOATS + (256 << 20)

    def _size_cache(self, kv_tokens: Optional[int], memory_ratio: float) -> int:
        """Pages of the cache: ``kv_tokens`` if given, else what ``memory_ratio`` of the free memory holds
        beside the per-request state and the step's workspace, at least 1024 tokens and at most eight
        contexts (src/engine.rs:317-329, src/model/mod.rs:406-439)."""
        if kv_tokens is None:
            free, _ = torch.cuda.mem_get_info(self.device)
            per_token = max(self._bytes_per_token(), 1)
            room = free * memory_ratio - self._workspace_bytes() - self._state_bytes()
            kv_tokens = int(max(room, 0) // per_token)
            kv_tokens = max(1024, min(kv_tokens, 8 * self.max_seq_len))
        return max(1, (int(kv_tokens) + self.page_size - 1) // self.page_size)

    # -- requests -------------------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[int] = None) -> int:
        params = params or SamplingParams()
        rid = self._next_id if request_id is None else int(request_id)
        self._next_id = max(self._next_id, rid) + 1
        self.scheduler.submit(rid, prompt_token_ids, params.max_tokens, params.ignore_eos, params.stop_token_ids)
        self._live[rid] = _Live(params, params.seed if params.seed is not None else fresh_seed(),
                                list(prompt_token_ids))
        return rid

    def abort(self, request_id: int) -> bool:
        return self.scheduler.abort(request_id)

    def has_unfinished(self) -> bool:
        return not self.scheduler.idle()

    def step(self) -> List[RequestOutput]:
        """Run one scheduler step; returns the requests that finished in it.

        While requests only decode, the step AFTER this one is launched before this one's tokens are read:
        it takes its token ids on the device from this step's picks, so the device goes from one step to
        the next without waiting for the host.  The next call then finds its step already running, launches
        the one after it, and only reads.  A request that ends on a token the host had not seen yet (an end
        token, an abort) has been computed one token too far; that token is dropped with the request."""
        flight, self._in_flight = self._in_flight, None
        self._last_error = None
        self.last_sampled = []
        plan = self.scheduler.plan_for(flight.ids) if flight is not None else []
        if not plan:                     # nothing on the device, or every request of it has ended meanwhile
            flight = None
            plan = self.scheduler.plan()
        if plan:
            try:
                if flight is None:
                    flight = self._launch(plan)
                else:
                    for e in plan:
                        if e.count != 1 or e.start != flight.starts[e.request_id]:
                            raise RuntimeError(f"request {e.request_id}: the step on the device is not the one planned")
                following = self._launch_following(flight, plan)
                tokens = self._read(flight, plan)
                self.runner.check_status()
                self.scheduler.commit(tokens)
                self._in_flight = following
                self.last_sampled = [(e.request_id, t, (self._live[e.request_id].logprobs[-1]
                                                        if self._live[e.request_id].params.logprobs > 0 else None))
                                     for e, t in zip((e for e in plan if e.sample), tokens)]
            except (StepError, KernelError, CacheError, torch.OutOfMemoryError) as exc:
                # the step failed on the device or for want of memory: its requests end with an error and
                # give their pages back, the others go on (src/scheduler.rs:1436-1463).  Anything else is
                # a fault of the program and is raised.
                self._last_error = str(exc)
                self.scheduler.fail_step()
        return self._collect()

    def _launch(self, plan, device_tokens: Optional[torch.Tensor] = None, steps_before: Optional[List[int]] = None):
        """Put a planned step on the device, its sampling and the copies that bring the picks back included.
        ``device_tokens``/``steps_before``: the step follows one whose picks are not on the host yet; its token
        ids come from that tensor, and request i has drawn ``steps_before[i]`` tokens before it."""
        entries = []
        for e in plan:
            live = self._live[e.request_id]
            if not live.adopted:
                self.runner.adopt_request(e.request_id)
                live.adopted = True
            entries.append(StepEntry(e.request_id, e.tokens, [e.count - 1] if e.sample else []))
        logits = self.runner.step(entries, device_tokens)
        flight = _InFlight([e.request_id for e in plan if e.sample],
                           {e.request_id: e.start for e in plan})
        if flight.ids:
            lives = [self._live[r] for r in flight.ids]
            plens = [len(l.prompt) for l in lives]
            generated = None
            if steps_before is not None:
                flight.steps = list(steps_before)
            elif any(l.params.has_penalties() for l in lives):       # token histories only where penalties read them
                outs = [self.scheduler.tokens_of(r) for r in flight.ids]
                flight.steps = [len(o) - p for o, p in zip(outs, plens)]
                generated = [o[p:] for o, p in zip(outs, plens)]
            else:
                flight.steps = [self.scheduler.num_tokens(r) - p for r, p in zip(flight.ids, plens)]
            flight.want_lp = [i for i, l in enumerate(lives) if l.params.logprobs > 0]
            flight.base = logits[flight.want_lp].cpu().numpy() if flight.want_lp else None    # before penalties
            flight.picks = self.sampler.sample(logits, [l.params for l in lives], [l.seed for l in lives], flight.steps,
                                               [l.prompt for l in lives], generated)
            flight.ticket = self.runner.begin_read_back(flight.picks)
        return flight

    def _launch_following(self, flight: "_InFlight", plan) -> Optional["_InFlight"]:
        """With ``flight`` on the device and unread: launch the step after it, if it is certain to be one more
        token for each of the same requests whatever ``flight`` picks short of an end token: every running
        request is in the plan and samples, nobody waits to be admitted, none ends by length.  Otherwise
        lay that step out on the host at least (if requests only decode), or do nothing."""
        decoding = all(e.sample for e in plan)
        lives = [self._live[e.request_id] for e in plan]
        if (self.run_ahead and decoding and len(plan) == len(flight.ids) and flight.ticket is not None
                and self.scheduler.waiting() == 0 and self.scheduler.running() == len(plan)
                and not any(l.params.has_penalties() or l.params.logprobs > 0 for l in lives)
                and all(self.scheduler.remaining(r) >= 2 for r in flight.ids)):
            nxt = [PlanEntry(e.request_id, e.slot, e.start + e.count, 1, True, [0]) for e in plan]
            try:
                following = self._launch(nxt, flight.picks, [s + 1 for s in flight.steps])
                self.run_ahead_steps += 1
                return following
            except (StepError, CacheError):
                return None                                     # the step itself will meet the same error, and report it
        if self.host_lookahead and decoding and all(e.count == 1 for e in plan):
            # the step is on its way: lay out the next one on the host while it runs
            self.runner.prepare_decode_ahead([e.request_id for e in plan])
        return None

    def _read(self, flight: "_InFlight", plan) -> List[int]:
        """Wait for ``flight`` and return the picks of the plan's sampled entries (the plan may have lost
        requests that ``flight`` still computed)."""
        if not flight.ids or flight.ticket is None:
            return []
        picks = self.runner.finish_read_back(flight.ticket)     # (waits for the step; the status word comes along)
        self.d2h_bytes_last = (len(picks) + 1) * 4
        for j, i in enumerate(flight.want_lp):
            live = self._live.get(flight.ids[i])
            if live is not None:
                live.logprobs.append(top_logprobs(flight.base[j], picks[i], live.params.logprobs))
        at = {r: i for i, r in enumerate(flight.ids)}
        return [picks[at[e.request_id]] for e in plan if e.sample]

    def _collect(self) -> List[RequestOutput]:
        out = []
        for rid, reason in self.scheduler.pop_finished():
            live = self._live.pop(rid)
            toks = self.scheduler.tokens_of(rid)
            n = len(live.prompt)
            err = None
            if reason == "error":
                err = self._last_error or "request does not fit in the KV cache"
            ro = RequestOutput(rid, toks[:n], toks[n:], reason, err, live.logprobs or None)
            self.scheduler.forget(rid)
            out.append(ro)
        return out

    def generate(self, prompt_token_ids: Sequence[Sequence[int]],
                 sampling_params: Union[None, SamplingParams, Sequence[SamplingParams]] = None) -> List[RequestOutput]:
        """Generate for a list of prompts (token ids in, token ids out), in the order given."""
        if prompt_token_ids and isinstance(prompt_token_ids[0], int):
            prompt_token_ids = [prompt_token_ids]      # one prompt
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompt_token_ids)
        ids, results = [], {}
        for prompt, sp in zip(prompt_token_ids, sampling_params):
            try:
                ids.append(self.add_request(prompt, sp))
            except SubmitError as exc:
                rid = self._next_id
                self._next_id += 1
                ids.append(rid)
                results[rid] = RequestOutput(rid, list(prompt), [], "error", str(exc))
        while self.has_unfinished():
            for ro in self.step():
                results[ro.request_id] = ro
        for ro in self._collect():
            results[ro.request_id] = ro
        return [results[i] for i in ids]

    def stats(self) -> Dict[str, int]:
        s = self.scheduler.stats()
        s["kv_pages_free"] = self.storage.manager.free_pages(0) if self.storage.groups else 0
        s["kv_pages_total"] = self.storage.groups[0].num_pages if self.storage.groups else 0
        return s
