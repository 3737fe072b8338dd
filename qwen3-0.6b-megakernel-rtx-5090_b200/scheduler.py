"""Continuous batching over the multi-sequence decode launch.

The reference serves one request at a time (a one-worker executor in ``megakernel.py:39``); its
benchmark configurations also name a continuous-batching mode.  This scheduler keeps up to
``engine.num_sequences`` requests live on one GPU.  Each round it

1. admits waiting requests into free slots in arrival order (the slot's KV cache is filled by the
   ``prefill`` op),
2. runs ONE persistent launch that advances every live sequence by ``q`` tokens, where ``q`` is the
   smaller of ``quantum`` and the fewest tokens any live sequence still needs (so no sequence runs past
   its budget and every launch ends on a point where a slot may free up),
3. cuts each sequence at EOS or at its budget, completes it and frees its slot.

The engine is any object with ``num_sequences``, ``max_seq_len``, ``prefill_slot(slot, ids)`` and
``decode_slots(slots, first_tokens, steps) -> list of token lists`` (``BatchDecoder`` provides them);
tests drive the scheduler with a fake engine on the CPU.

``overlap_prefill=True`` moves step 1 to its own thread: while a decode launch of the live sequences runs, the
next waiting request is prefilled into a free slot (the engine must allow ``prefill_slot`` of one slot to run
concurrently with ``decode_slots`` of others; ``BatchDecoder`` with the tensor-core engines does, on separate
CUDA streams and workspaces).  A slot joins the next decode round after its prefill has finished.
"""

from __future__ import annotations

import threading
from collections import deque
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence


@dataclass
class Request:
    rid: int
    prompt_ids: List[int]
    max_tokens: int
    future: Future = field(default_factory=Future, repr=False)
    # filled while the request is live
    slot: int = -1
    next_token: int = -1           # input token of the next decode step
    out: List[int] = field(default_factory=list)


@dataclass
class Result:
    rid: int
    tokens: List[int]
    prompt_tokens: int
    finish_reason: str             # "stop" (EOS) or "length"


class ContinuousBatcher:
    def __init__(self, engine, eos_token_id: Optional[int] = None, quantum: int = 16, overlap_prefill: bool = False,
                 packed_prefill: bool = True, live_limit: Optional[int] = None):
        if quantum < 1:
            raise ValueError("quantum must be >= 1")
        if live_limit is not None and live_limit < 1:
            raise ValueError("live_limit must be >= 1")
        self.engine = engine
        self.overlap_prefill = bool(overlap_prefill)
        # several waiting requests per prefill pass where the engine offers it; False: one pass per request (a
        # request's cache then does not depend on who was admitted with it, not even in the last bits)
        self.packed_prefill = bool(packed_prefill)
        self._prefilling = 0                          # requests taken from the queue whose prefill is running
        self._admit_thread: Optional[threading.Thread] = None
        self.eos = -1 if eos_token_id is None else int(eos_token_id)
        self.quantum = int(quantum)
        self.num_slots = int(engine.num_sequences)
        # at most this many sequences decode together; the engine's other slots hold requests that are prefilled already
        # and take a seat in the round after one frees up (without them a seat stays empty for a round while its next
        # request is prefilled)
        self.live_limit = self.num_slots if live_limit is None else min(int(live_limit), self.num_slots)
        self._ready: Deque[Request] = deque()         # prefilled, waiting for a seat
        self._waiting: Deque[Request] = deque()
        self._live: Dict[int, Request] = {}           # slot -> request
        self._free: List[int] = list(range(self.num_slots))
        self._lock = threading.Lock()
        self._wake = threading.Condition(self._lock)
        self._next_id = 0
        self._thread: Optional[threading.Thread] = None
        self._stop = False
        self._admit_stop = False
        # counters for tests and reports
        self.launches = 0
        self.decoded_tokens = 0        # tokens produced by launches, including ones cut after EOS
        self.max_live = 0

    # ------------------------------------------------------------------ submission
    def submit(self, prompt_ids: Sequence[int], max_tokens: int) -> Future:
        """Queue a request; the future resolves to a ``Result`` (or raises what the engine raised)."""
        ids = [int(t) for t in prompt_ids]
        req = Request(rid=-1, prompt_ids=ids, max_tokens=int(max_tokens))
        if not ids:
            req.future.set_exception(ValueError("empty prompt"))
            return req.future
        if len(ids) - 1 + max(req.max_tokens, 0) > self.engine.max_seq_len:
            req.future.set_exception(ValueError("prompt + max_tokens exceeds max_seq_len"))
            return req.future
        with self._wake:
            req.rid = self._next_id
            self._next_id += 1
            if req.max_tokens <= 0:
                req.future.set_result(Result(req.rid, [], len(ids), "length"))
                return req.future
            self._waiting.append(req)
            self._wake.notify_all()
        return req.future

    # ------------------------------------------------------------------ one scheduling round
    def _admit(self) -> None:
        """Prefills waiting requests into free slots until one of the two runs out.  An engine with ``prefill_slots``
        (several prompts in one pass, up to ``packed_prefill_rows`` rows after padding each to a multiple of 128)
        gets every waiting request that fits at once: a pass over one ~1000-token prompt is mostly launch latency."""
        packed = getattr(self.engine, "prefill_slots", None) if self.packed_prefill else None
        budget = int(getattr(self.engine, "packed_prefill_rows", 0)) if packed is not None else 0
        while True:
            with self._wake:
                if not self._waiting or not self._free:
                    return
                group = []
                rows = 0
                while self._waiting and self._free and len(group) < 64:
                    need = (max(len(self._waiting[0].prompt_ids) - 1, 1) + 127) // 128 * 128
                    if group and (budget <= 0 or rows + need > budget):
                        break
                    rows += need
                    group.append((self._waiting.popleft(), self._free.pop(0)))
                    if budget <= 0:
                        break
                self._prefilling += len(group)
            if len(group) > 1:
                try:
                    packed([slot for _, slot in group], [req.prompt_ids[:-1] for req, _ in group])
                    failed = {}
                except Exception:              # find the culprit: fall back to one pass per request
                    failed = None
            else:
                failed = None
            if failed is None:
                failed = {}
                for req, slot in group:
                    try:
                        self.engine.prefill_slot(slot, req.prompt_ids[:-1])
                    except Exception as exc:   # a bad prompt fails its own request only
                        failed[slot] = exc
            with self._wake:
                for req, slot in group:
                    self._prefilling -= 1
                    if slot in failed:
                        self._free.append(slot)
                        self._free.sort()
                    else:
                        req.slot = slot
                        req.next_token = req.prompt_ids[-1]
                        self._ready.append(req)
                self._wake.notify_all()
            for req, slot in group:
                if slot in failed:
                    req.future.set_exception(failed[slot])

    def step(self) -> bool:
        """One round (admit, launch, retire).  Returns False when there was nothing to do."""
        if self.overlap_prefill:
            self._ensure_admit_thread()
            with self._wake:                   # nothing live yet but a prefill is on its way: wait for it
                while not self._live and not self._ready and (self._prefilling or (self._waiting and self._free)):
                    self._wake.wait(timeout=0.05)
        else:
            self._admit()
        with self._lock:
            while self._ready and len(self._live) < self.live_limit:
                r = self._ready.popleft()
                self._live[r.slot] = r
            self.max_live = max(self.max_live, len(self._live))
            live = [self._live[s] for s in sorted(self._live)]
        if not live:
            return False
        q = min(self.quantum, min(r.max_tokens - len(r.out) for r in live))
        slots = [r.slot for r in live]
        try:
            produced = self.engine.decode_slots(slots, [r.next_token for r in live], q)
        except Exception as exc:               # an engine failure ends every live request
            with self._lock:
                for r in live:
                    del self._live[r.slot]
                    self._free.append(r.slot)
                self._free.sort()
            for r in live:
                r.future.set_exception(exc)
            return True
        self.launches += 1
        self.decoded_tokens += q * len(live)
        for r, toks in zip(live, produced):
            finish = None
            for t in toks:
                if t == self.eos:
                    finish = "stop"
                    break
                r.out.append(int(t))
            if finish is None and len(r.out) >= r.max_tokens:
                finish = "length"
            if finish is None:
                r.next_token = int(toks[-1])
                continue
            with self._wake:
                del self._live[r.slot]
                self._free.append(r.slot)
                self._free.sort()
                self._wake.notify_all()        # the admission thread may be waiting for a slot
            r.future.set_result(Result(r.rid, r.out, len(r.prompt_ids), finish))
        return True

    # ------------------------------------------------------------------ overlapped admission
    def _ensure_admit_thread(self) -> None:
        if self._admit_thread is None or not self._admit_thread.is_alive():
            self._admit_stop = False
            self._admit_thread = threading.Thread(target=self._admit_loop, name="batcher-prefill", daemon=True)
            self._admit_thread.start()

    def _admit_loop(self) -> None:
        while True:
            self._admit()
            with self._wake:
                if self._admit_stop:
                    return
                if not (self._waiting and self._free):
                    self._wake.wait(timeout=0.05)

    def run_until_idle(self) -> None:
        """Synchronous driver: rounds until no request is waiting, being prefilled or live."""
        while True:
            if self.step():
                continue
            with self._lock:
                if not self._waiting and not self._live and not self._prefilling and not self._ready:
                    return

    # ------------------------------------------------------------------ background driver
    def start(self) -> None:
        if self._thread is not None:
            return
        self._stop = False
        self._thread = threading.Thread(target=self._loop, name="continuous-batcher", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        with self._wake:
            self._stop = True
            self._wake.notify_all()
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._admit_thread is not None:
            with self._wake:
                self._admit_stop = True
                self._wake.notify_all()
            self._admit_thread.join()
            self._admit_thread = None

    def _loop(self) -> None:
        while True:
            if not self.step():
                with self._wake:
                    if self._stop:
                        return
                    if not self._waiting and not self._live and not self._prefilling and not self._ready:
                        self._wake.wait(timeout=0.5)
            with self._lock:
                if self._stop and not self._waiting and not self._live and not self._prefilling and not self._ready:
                    return
