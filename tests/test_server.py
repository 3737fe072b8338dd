"""CPU tests of the OpenAI-style server and the load generator with a stub decoder (no GPU, no checkpoint)."""

import pytest

fastapi = pytest.importorskip("fastapi")
from starlette.testclient import TestClient  # noqa: E402

import loadgen  # noqa: E402
import server  # noqa: E402
import synthetic as S  # noqa: E402


class FakeDecoder:
    """Echo model: answers with the prompt's ids + 1, at most max_tokens of them; stops early on id 7."""

    def __init__(self):
        self.tokenizer = S.StubTokenizer(eos_token_id=7, vocab_size=1000)
        self.prompts = []

    def generate(self, prompt, max_tokens=100):
        self.prompts.append(prompt)
        ids = self.tokenizer.encode(prompt)
        out = []
        for t in ids[:max_tokens]:
            if t + 1 == 7:
                break
            out.append(t + 1)
        return self.tokenizer.decode(out), len(ids), len(out)


class ThinkTokenizer(S.StubTokenizer):
    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True):
        return "<think>\nplan\n</think>\n\n" + " ".join(m["content"] for m in messages) + "  \n"


@pytest.fixture()
def client():
    dec = FakeDecoder()
    app = server.create_app(decoder=dec, model_name="stub-model", default_max_tokens=5)
    with TestClient(app) as c:
        c.decoder = dec
        yield c


def test_health_and_models(client):
    assert client.get("/health").json() == {"status": "ok"}
    m = client.get("/v1/models").json()
    assert m["object"] == "list" and m["data"][0]["id"] == "stub-model" and m["data"][0]["owned_by"] == "megakernel"


def test_chat_completion_schema_and_usage(client):
    r = client.post("/v1/chat/completions", json={"model": "x", "messages": [{"role": "user", "content": "10 20 30"}],
                                                  "max_tokens": 8, "temperature": 0.7, "stream": True})
    assert r.status_code == 200
    body = r.json()
    assert body["object"] == "chat.completion" and body["id"].startswith("chatcmpl-") and body["model"] == "stub-model"
    choice = body["choices"][0]
    assert choice["index"] == 0 and choice["message"] == {"role": "assistant", "content": "11 21 31"}
    assert choice["finish_reason"] == "stop"                        # fewer tokens than the budget
    assert body["usage"] == {"prompt_tokens": 3, "completion_tokens": 3, "total_tokens": 6}
    r2 = client.post("/v1/chat/completions", json={"model": "x", "messages": [{"role": "user", "content": "1 2 3 4"}],
                                                   "max_tokens": 2})
    assert r2.json()["choices"][0]["finish_reason"] == "length"      # budget exhausted
    assert r2.json()["id"] != body["id"]


def test_prompt_building_suppresses_thinking():
    msgs = [server.Message(role="user", content="5 6")]
    p = server.build_prompt(ThinkTokenizer(), msgs)
    assert p == "5 6\n<think>\n\n</think>\n\n"


def test_engine_errors_become_http_500():
    class Broken(FakeDecoder):
        def generate(self, prompt, max_tokens=100):
            raise RuntimeError("device status 4")
    with TestClient(server.create_app(decoder=Broken(), model_name="m")) as c:
        r = c.post("/v1/chat/completions", json={"model": "m", "messages": [{"role": "user", "content": "1"}]})
        assert r.status_code == 500 and "device status 4" in r.json()["detail"]


def test_load_env(tmp_path, monkeypatch):
    f = tmp_path / ".env"
    f.write_text("# comment\nPORT=9001\nMODEL = my/model\nBROKEN\n")
    monkeypatch.delenv("PORT", raising=False)
    monkeypatch.setenv("MODEL", "kept")
    server.load_env(str(f))
    import os
    assert os.environ["PORT"] == "9001" and os.environ["MODEL"] == "kept"


def test_load_generator_against_the_app(client):
    prompts = loadgen.synthetic_prompts(6, 4, seed=1, vocab=500)
    assert prompts == loadgen.synthetic_prompts(6, 4, seed=1, vocab=500) and len(prompts[0].split()) == 4
    post = lambda body: client.post("/v1/chat/completions", json=body).json()
    rep = loadgen.run(post, prompts, model="stub-model", max_tokens=3, concurrency=2)
    s = rep["summary"]
    assert s["num_requests"] == 6 and s["num_failed"] == 0
    for k in ("avg_latency_s", "median_latency_s", "std_latency_s", "min_latency_s", "max_latency_s",
              "throughput_req_s", "tokens_per_s"):
        assert k in s
    assert s["min_latency_s"] <= s["median_latency_s"] <= s["max_latency_s"]
    assert all(r["output_tokens"] <= 3 for r in rep["results"])
    bad = loadgen.run(lambda body: (_ for _ in ()).throw(RuntimeError("down")), prompts[:2], "m", 3)
    assert bad["summary"]["num_failed"] == 2 and bad["summary"]["avg_latency_s"] == 0.0


@pytest.mark.gpu
def test_server_end_to_end_on_the_engine(built_library):
    """The real Decoder (tiny seeded model, stub tokenizer) behind the HTTP surface: the answer is the oracle's
    greedy continuation of the prompt's ids."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from Model.Qwen06B_architecture import Decoder
    from oracle.decoder_ref import Decoder as Oracle
    w = S.make_weights(seed=3, num_layers=2, vocab_size=4096, norm_std=0.1, max_seq_len=64)
    ids = S.make_prompt(12, seed=5, vocab_size=4096)
    want, _ = Oracle(w, max_seq_len=64).generate_ids(ids, 6)
    dec = Decoder(weights=S.weights_to(w, "cuda"), tokenizer=S.StubTokenizer(-1, 4096), verbose=False, max_seq_len=64)
    with TestClient(server.create_app(decoder=dec, model_name="tiny")) as c:
        r = c.post("/v1/chat/completions", json={"model": "tiny", "max_tokens": 6,
                                                 "messages": [{"role": "user", "content": " ".join(map(str, ids))}]})
        assert r.status_code == 200, r.text
        body = r.json()
        assert body["choices"][0]["message"]["content"] == " ".join(map(str, want))
        assert body["choices"][0]["finish_reason"] == "length"
        assert body["usage"] == {"prompt_tokens": 12, "completion_tokens": 6, "total_tokens": 18}
        rep = loadgen.run(lambda b: c.post("/v1/chat/completions", json=b).json(),
                          loadgen.synthetic_prompts(4, 8, seed=2, vocab=4096), "tiny", 4)
        assert rep["summary"]["num_failed"] == 0 and rep["summary"]["tokens_per_s"] > 0


def test_batching_mode_serves_concurrent_requests_with_real_finish_reason():
    """A multi-sequence engine behind the app: requests go through the continuous-batching scheduler,
    several are live at once, and finish_reason says whether EOS or the budget ended the answer."""
    from concurrent.futures import ThreadPoolExecutor
    from test_scheduler import FakeEngine

    eng = FakeEngine(num_sequences=3, max_seq_len=128)
    ids, budget = [5, 9, 2], 12
    full, _ = FakeEngine.reference(ids, budget)
    eng.tokenizer = S.StubTokenizer(eos_token_id=full[6], vocab_size=97)
    app = server.create_app(decoder=eng, model_name="stub-batch", default_max_tokens=4)
    with TestClient(app) as c:
        def ask(content, max_tokens):
            return c.post("/v1/chat/completions", json={"model": "x", "messages": [{"role": "user", "content": content}],
                                                        "max_tokens": max_tokens}).json()
        with ThreadPoolExecutor(6) as pool:
            futs = [pool.submit(ask, "5 9 2", budget)] + [pool.submit(ask, f"{i} {i + 1}", 3 + i) for i in range(5)]
            bodies = [f.result() for f in futs]
        stop = bodies[0]
        assert stop["choices"][0]["finish_reason"] == "stop"
        assert stop["choices"][0]["message"]["content"] == " ".join(map(str, full[:6]))
        assert stop["usage"] == {"prompt_tokens": 3, "completion_tokens": 6, "total_tokens": 9}
        for i, b in enumerate(bodies[1:]):
            want, why = FakeEngine.reference([i, i + 1], 3 + i, full[6])
            assert b["choices"][0]["message"]["content"] == " ".join(map(str, want))
            assert b["choices"][0]["finish_reason"] == why
        assert app.state.engine["batcher"].launches > 0
