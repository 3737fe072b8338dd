"""OpenAI-style chat-completions server on top of the B200 ``Decoder``.

Same surface as the reference server (``Tools/megakernel/megakernel.py``): ``GET /health``
(:90-92), ``GET /v1/models`` (:95-101), ``POST /v1/chat/completions`` (:121-153) with the request
fields ``model, messages, max_tokens, temperature, stream``; ``.env`` / environment keys ``PORT``,
``MODEL``, ``MAX_TOKENS`` (:10-27); prompts built from the tokenizer's chat template with Qwen3
thinking suppressed (:104-113); one decode at a time (the engine is single-stream per GPU, :39).
``temperature`` and ``stream`` are accepted and ignored, as there (greedy, non-streaming).

Differences: ``finish_reason`` is "length" when the token budget was exhausted and "stop" when the
model emitted EOS (the reference always says "stop"); the app is built by ``create_app`` so a test can
inject a decoder; ``SYNTHETIC=1`` serves a seeded random-weight model with the decimal-ID stub tokenizer
(no checkpoint is needed to bring the server up).
"""

from __future__ import annotations

import asyncio
import itertools
import os
import re
import sys
import time
from concurrent.futures import ThreadPoolExecutor
from contextlib import asynccontextmanager
from pathlib import Path
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)


def load_env(path: str = ".env") -> None:
    """KEY=VALUE lines of a .env file into os.environ (existing variables win)."""
    f = Path(path)
    if not f.is_file():
        return
    for raw in f.read_text().splitlines():
        line = raw.strip()
        if line and not line.startswith("#") and "=" in line:
            k, v = line.split("=", 1)
            os.environ.setdefault(k.strip(), v.strip())


from fastapi import FastAPI, HTTPException  # noqa: E402
from pydantic import BaseModel  # noqa: E402

_THINK_BLOCK = re.compile(r"<think>.*?</think>\n*", re.DOTALL)
_EMPTY_THINK = "\n<think>\n\n</think>\n\n"


class Message(BaseModel):
    role: str
    content: str


class ChatRequest(BaseModel):
    model: str
    messages: List[Message]
    max_tokens: Optional[int] = 128
    temperature: Optional[float] = 0.0
    stream: Optional[bool] = False


def build_prompt(tokenizer, messages: List[Message]) -> str:
    """Chat template + generation prompt, any think block removed and an empty one appended so the
    model answers directly (reference: megakernel.py:104-113)."""
    msgs = [{"role": m.role, "content": m.content} for m in messages]
    text = tokenizer.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True)
    return _THINK_BLOCK.sub("", text).rstrip() + _EMPTY_THINK


def _load_decoder(model_name: str):
    """``BATCH_SLOTS`` > 1 (up to 128; above 4 the tensor-core batched decode) loads the multi-sequence
    engine: requests are then served concurrently by the continuous-batching scheduler, with tensor-core
    prefill (several waiting prompts per pass), instead of one at a time.  ``BATCH_LIVE`` (optional, below
    ``BATCH_SLOTS``) caps the sequences that decode together; the remaining slots are prefilled ahead."""
    from Model.Qwen06B_architecture import BatchDecoder, Decoder, load_weights
    slots = int(os.getenv("BATCH_SLOTS", "1"))
    if os.getenv("SYNTHETIC", "0") == "1":
        import synthetic as S
        layers = int(os.getenv("SYNTHETIC_LAYERS", "28"))
        w = S.weights_to(S.make_weights(seed=0, num_layers=layers), "cuda")
        tok = S.StubTokenizer(eos_token_id=-1)
    elif slots > 1:
        w, tok = load_weights(model_name, verbose=True)
    else:
        return Decoder(model_name=model_name, verbose=True)
    if slots > 1:
        return BatchDecoder(weights=w, tokenizer=tok, num_sequences=slots, verbose=False, prefill_mode="tensor")
    return Decoder(weights=w, tokenizer=tok, verbose=False)


def create_app(decoder=None, model_name: Optional[str] = None, default_max_tokens: Optional[int] = None) -> FastAPI:
    model_name = model_name or os.getenv("MODEL", "Qwen/Qwen3-0.6B")
    default_max_tokens = default_max_tokens or int(os.getenv("MAX_TOKENS", "128"))
    state = {"decoder": decoder, "batcher": None}
    worker = ThreadPoolExecutor(max_workers=1)      # single-sequence engine: one request at a time per GPU
    ids = itertools.count(1)

    def start_batcher():
        dec = state["decoder"]
        if state["batcher"] is None and hasattr(dec, "decode_slots"):   # multi-sequence engine
            from scheduler import ContinuousBatcher
            eos = getattr(dec.tokenizer, "eos_token_id", None)
            # BATCH_LIVE < BATCH_SLOTS: that many sequences decode together, the other slots hold prefilled requests
            live = int(os.getenv("BATCH_LIVE", "0"))
            state["batcher"] = ContinuousBatcher(dec, eos_token_id=eos, quantum=int(os.getenv("BATCH_QUANTUM", "16")),
                                                 overlap_prefill=getattr(dec, "supports_overlap", False),
                                                 live_limit=live if live > 0 else None)
            state["batcher"].start()

    @asynccontextmanager
    async def lifespan(app: FastAPI):
        if state["decoder"] is None:
            t0 = time.time()
            print(f"[server] loading {model_name} ...", flush=True)
            state["decoder"] = _load_decoder(model_name)
            print(f"[server] ready in {time.time() - t0:.1f}s", flush=True)
        start_batcher()
        yield
        if state["batcher"] is not None:
            state["batcher"].stop()
        worker.shutdown(wait=False)

    app = FastAPI(title="Qwen3-0.6B B200 megakernel server", lifespan=lifespan)
    app.state.engine = state

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list",
                "data": [{"id": model_name, "object": "model", "created": int(time.time()), "owned_by": "megakernel"}]}

    def run(messages: List[Message], budget: int):
        dec = state["decoder"]
        prompt = build_prompt(dec.tokenizer, messages)
        return dec.generate(prompt, max_tokens=budget)

    @app.post("/v1/chat/completions")
    async def chat_completions(req: ChatRequest):
        if state["decoder"] is None:
            raise HTTPException(status_code=503, detail="Model not loaded yet")
        budget = req.max_tokens or default_max_tokens
        finish = None
        try:
            if state["batcher"] is not None:
                dec = state["decoder"]
                prompt_ids = dec.tokenizer.encode(build_prompt(dec.tokenizer, req.messages), add_special_tokens=False)
                res = await asyncio.wrap_future(state["batcher"].submit(prompt_ids, budget))
                text = dec.tokenizer.decode(res.tokens, skip_special_tokens=True)
                n_in, n_out, finish = res.prompt_tokens, len(res.tokens), res.finish_reason
            else:
                text, n_in, n_out = await asyncio.get_running_loop().run_in_executor(worker, run, req.messages, budget)
        except Exception as exc:  # engine errors surface as HTTP 500 with the engine's message
            raise HTTPException(status_code=500, detail=str(exc))
        return {
            "id": f"chatcmpl-{next(ids)}",
            "object": "chat.completion",
            "created": int(time.time()),
            "model": model_name,
            "choices": [{"index": 0, "message": {"role": "assistant", "content": text},
                         "finish_reason": finish or ("length" if n_out >= budget else "stop")}],
            "usage": {"prompt_tokens": n_in, "completion_tokens": n_out, "total_tokens": n_in + n_out},
        }

    return app


if __name__ == "__main__":
    import uvicorn
    load_env()
    uvicorn.run(create_app(), host="0.0.0.0", port=int(os.getenv("PORT", "8000")), log_level="warning",
                access_log=False)
