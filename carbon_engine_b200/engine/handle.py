"""The engine behind a thread of its own: requests go in through a command queue, tokens come back as
events while the next step already runs.

This is the shape of the reference's ``scheduler::spawn`` + ``EngineHandle`` (src/scheduler.rs:190-251,
385-473): the scheduler loop owns the engine; ``submit`` returns at once with the request's id and a
stream of events (``Token`` ... then ``Done`` or ``Error``, src/scheduler.rs:1421-1433, 1551-1581);
``abort`` and ``stats`` are commands like any other.  The loop blocks on the queue while idle, and
between two steps takes whatever commands have arrived.  ``Engine.generate`` remains the synchronous
way for tests and scripts.
"""
from __future__ import annotations

import queue
import threading
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Sequence, Union

from ..sampling.params import SamplingParams
from .scheduler import SubmitError


@dataclass(frozen=True)
class Token:
    token_id: int


@dataclass(frozen=True)
class Logprobs:
    entry: dict            # {"token", "logprob", "top": [(token, logprob), ...]} of the token that follows


@dataclass(frozen=True)
class Done:
    reason: str            # "stop", "length" or "abort"
    usage: Dict[str, int]  # prompt_tokens, completion_tokens


@dataclass(frozen=True)
class Error:
    message: str


Event = Union[Token, Logprobs, Done, Error]


class RequestStream:
    """The events of one request, in order; iteration ends after ``Done`` or ``Error``."""

    def __init__(self, request_id: int):
        self.request_id = request_id
        self._events: "queue.Queue[Event]" = queue.Queue()
        self._ended = False

    def get(self, timeout: Optional[float] = None) -> Event:
        ev = self._events.get(timeout=timeout)
        if isinstance(ev, (Done, Error)):
            self._ended = True
        return ev

    def __iter__(self) -> Iterator[Event]:
        while not self._ended:
            yield self.get()

    def collect(self, timeout: Optional[float] = None):
        """Wait for the end: (token ids, the final ``Done`` or ``Error``)."""
        toks: List[int] = []
        while True:
            ev = self.get(timeout)
            if isinstance(ev, Token):
                toks.append(ev.token_id)
            elif isinstance(ev, (Done, Error)):
                return toks, ev


class EngineHandle:
    """Owns an :class:`Engine` on a thread; safe to call from any thread."""

    def __init__(self, engine):
        self.engine = engine
        self._commands: "queue.Queue[tuple]" = queue.Queue()
        self._streams: Dict[int, RequestStream] = {}
        self._next_id = 0
        self._id_lock = threading.Lock()
        self._stopped = threading.Event()
        self._thread = threading.Thread(target=self._run, name="carbon-scheduler", daemon=True)
        self._thread.start()

    # -- the caller's side ------------------------------------------------------------------------
    def submit(self, prompt_token_ids: Sequence[int], params: Optional[SamplingParams] = None) -> RequestStream:
        with self._id_lock:
            rid = self._next_id
            self._next_id += 1
        stream = RequestStream(rid)
        if self._stopped.is_set():
            stream._events.put(Error("engine is not running"))
        else:
            self._commands.put(("submit", stream, list(prompt_token_ids), params or SamplingParams()))
        return stream

    def abort(self, request_id: int) -> None:
        self._commands.put(("abort", request_id))

    def stats(self, timeout: Optional[float] = 60.0) -> Optional[dict]:
        if self._stopped.is_set():
            return None
        reply: "queue.Queue[dict]" = queue.Queue()
        self._commands.put(("stats", reply))
        try:
            return reply.get(timeout=timeout)
        except queue.Empty:
            return None

    def shutdown(self) -> None:
        """Stop the loop after the step in flight; requests still running end with an error."""
        if not self._stopped.is_set():
            self._commands.put(("stop",))
        self._thread.join()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.shutdown()

    # -- the scheduler thread ---------------------------------------------------------------------
    def _run(self) -> None:
        import torch
        torch.cuda.set_device(self.engine.device)
        eng = self.engine
        try:
            while True:
                # idle: sleep on the queue; busy: take what has arrived and go on stepping
                block = not eng.has_unfinished()
                while True:
                    try:
                        cmd = self._commands.get(block=block)
                    except queue.Empty:
                        break
                    block = False
                    if cmd[0] == "stop":
                        return
                    self._handle(cmd)
                if not eng.has_unfinished():
                    self._flush(eng._collect())
                    continue
                finished = eng.step()
                for rid, tok, lp in eng.last_sampled:
                    stream = self._streams.get(rid)
                    if stream is not None:
                        if lp is not None:
                            stream._events.put(Logprobs(lp))
                        stream._events.put(Token(tok))
                self._flush(finished)
        except BaseException as exc:      # a fault of the program: tell every waiting caller, then stop
            for stream in self._streams.values():
                stream._events.put(Error(f"engine stopped: {exc!r}"))
            self._streams.clear()
            raise
        finally:
            self._stopped.set()
            for stream in self._streams.values():
                stream._events.put(Error("engine is not running"))
            self._streams.clear()
            while True:                    # commands that were never taken
                try:
                    cmd = self._commands.get_nowait()
                except queue.Empty:
                    break
                if cmd[0] == "submit":
                    cmd[1]._events.put(Error("engine is not running"))
                elif cmd[0] == "stats":
                    cmd[1].put({})

    def _handle(self, cmd: tuple) -> None:
        eng = self.engine
        if cmd[0] == "submit":
            _, stream, prompt, params = cmd
            try:
                eng.add_request(prompt, params, request_id=stream.request_id)
            except SubmitError as exc:
                stream._events.put(Error(str(exc)))
                return
            self._streams[stream.request_id] = stream
        elif cmd[0] == "abort":
            eng.abort(cmd[1])
        elif cmd[0] == "stats":
            cmd[1].put(eng.stats())

    def _flush(self, finished) -> None:
        for out in finished:
            stream = self._streams.pop(out.request_id, None)
            if stream is None:
                continue
            if out.finish_reason == "error":
                stream._events.put(Error(out.error or "the step failed"))
            else:
                stream._events.put(Done(out.finish_reason, out.usage))
