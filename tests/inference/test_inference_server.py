"""OpenAI-compatible server through FastAPI's test client: endpoints, batching, logprobs, n > 1, weight reload."""
import threading

import pytest
import torch

fastapi = pytest.importorskip("fastapi")
from fastapi.testclient import TestClient  # noqa: E402

from levanter_b200.inference.engine import InferenceEngineConfig  # noqa: E402
from levanter_b200.inference.openai import InferenceServer, InferenceServerConfig  # noqa: E402
from levanter_b200.models.llama import LlamaConfig  # noqa: E402


class CharTokenizer:
    """Bytes as tokens; enough of the Hugging Face interface for the server."""
    eos_token_id = 0
    bos_token_id = None
    pad_token_id = 0
    chat_template = None

    def __call__(self, text, add_special_tokens=False, **kw):
        return {"input_ids": list(text.encode("utf-8"))}

    def decode(self, ids, skip_special_tokens=True):
        return bytes(int(i) % 256 for i in ids if not (skip_special_tokens and int(i) == 0)).decode("latin-1")

    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=True):
        raise ValueError("no chat template")

    def __len__(self):
        return 256


@pytest.fixture(scope="module")
def server():
    model = LlamaConfig(seq_len=128, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, num_kv_heads=2).build(256, seed=0).eval()
    cfg = InferenceServerConfig(service=InferenceEngineConfig(max_seqs=4, page_size=8, max_pages_per_seq=8, compute_dtype=torch.float32,
                                                              max_rounds=4, enable_logprobs=True), batch_timeout=0.02)
    srv = InferenceServer.create(cfg, model=model, tokenizer=CharTokenizer())
    yield srv
    srv.shutdown()


def test_endpoints_and_short_request(server):
    with TestClient(server.app) as client:
        assert client.get("/health").json()["status"] == "healthy"
        r = client.post("/v1/completions", json={"model": "m", "prompt": "hello", "max_tokens": 5, "temperature": 0.0})
        assert r.status_code == 200, r.text
        body = r.json()
        assert body["object"] == "text_completion" and len(body["choices"]) == 1
        assert body["usage"]["prompt_tokens"] == 5 and 1 <= body["usage"]["completion_tokens"] <= 5
        r2 = client.post("/v1/completions", json={"model": "m", "prompt": "hello", "max_tokens": 5, "temperature": 0.0})
        assert r2.json()["choices"][0]["text"] == body["choices"][0]["text"]  # greedy decoding is deterministic


def test_logprobs_n_and_chat(server):
    with TestClient(server.app) as client:
        r = client.post("/v1/completions", json={"model": "m", "prompt": "abc", "max_tokens": 4, "temperature": 0.8, "n": 3, "logprobs": 1, "seed": 5})
        body = r.json()
        assert len(body["choices"]) == 3
        for c in body["choices"]:
            lp = c["logprobs"]["token_logprobs"]
            assert 1 <= len(lp) <= 4 and all(x <= 0 for x in lp)
        again = client.post("/v1/completions", json={"model": "m", "prompt": "abc", "max_tokens": 4, "temperature": 0.8, "n": 3, "logprobs": 1, "seed": 5})
        assert [c["text"] for c in again.json()["choices"]] == [c["text"] for c in body["choices"]]
        chat = client.post("/v1/chat/completions", json={"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 3,
                                                         "temperature": 0.0, "logprobs": True})
        cb = chat.json()
        assert chat.status_code == 200 and cb["choices"][0]["message"]["role"] == "assistant"
        assert len(cb["choices"][0]["logprobs"]["content"]) == cb["usage"]["completion_tokens"]


def test_logprobs_are_reproducible_and_differ_between_generations(server):
    with TestClient(server.app) as client:
        req = {"model": "m", "prompt": "Once upon a time", "max_tokens": 4, "temperature": 0.0, "logprobs": True, "seed": 12345}
        a, b = (client.post("/v1/completions", json=req).json()["choices"][0]["logprobs"] for _ in range(2))
        assert a["tokens"] == b["tokens"] and len(a["tokens"]) == len(a["token_logprobs"]) > 0
        assert all(abs(x - y) < 1e-6 for x, y in zip(a["token_logprobs"], b["token_logprobs"]))
        two = client.post("/v1/completions", json={"model": "m", "prompt": "One plus one is", "max_tokens": 10, "temperature": 0.7,
                                                   "logprobs": True, "n": 2, "seed": 42}).json()["choices"]
        assert [c["index"] for c in two] == [0, 1]
        assert two[0]["logprobs"]["token_logprobs"] != two[1]["logprobs"]["token_logprobs"]  # the clones sample independently


def test_reload_with_zeroed_weights_and_back(server):
    import copy

    with TestClient(server.app) as client:
        req = {"model": "m", "prompt": "The quick brown fox", "max_tokens": 16, "temperature": 0.0, "seed": 42}
        original = client.post("/v1/completions", json=req).json()
        kept = {}

        def zero(model):
            kept["state"] = copy.deepcopy(model.state_dict())
            with torch.no_grad():
                for p in model.parameters():
                    p.zero_()
            return model

        server.reload(zero)
        zeroed = client.post("/v1/completions", json=req).json()
        assert zeroed["usage"]["completion_tokens"] > 0
        # all logits equal: greedy decoding picks token 0 = end of sequence at once, or at least something else than before
        assert zeroed["choices"][0]["text"] != original["choices"][0]["text"] or original["usage"]["completion_tokens"] == 1

        def restore(model):
            model.load_state_dict(kept["state"])
            return model

        server.reload(restore)
        assert client.post("/v1/completions", json=req).json()["choices"][0]["text"] == original["choices"][0]["text"]


def test_too_long_request_is_a_400(server):
    with TestClient(server.app) as client:
        r = client.post("/v1/completions", json={"model": "m", "prompt": "x" * 60, "max_tokens": 50})
        assert r.status_code == 400
        r = client.post("/v1/completions", json={"model": "m", "prompt": "x", "max_tokens": 4, "stream": True})
        assert r.status_code == 400


def test_weight_reload_during_requests(server):
    with TestClient(server.app) as client:
        before = client.post("/v1/completions", json={"model": "m", "prompt": "reload", "max_tokens": 6, "temperature": 0.0}).json()
        results = []

        def fire():
            results.append(client.post("/v1/completions", json={"model": "m", "prompt": "reload", "max_tokens": 6, "temperature": 0.0}).status_code)

        threads = [threading.Thread(target=fire) for _ in range(4)]
        for t in threads:
            t.start()

        def new_weights(model):
            with torch.no_grad():
                for p in model.parameters():
                    p.add_(torch.randn_like(p) * 0.5)
            return model

        server.reload(new_weights)
        for t in threads:
            t.join()
        assert results == [200] * 4
        after = client.post("/v1/completions", json={"model": "m", "prompt": "reload", "max_tokens": 6, "temperature": 0.0}).json()
        assert after["choices"][0]["text"] != before["choices"][0]["text"]
        server.unload()
        assert client.post("/v1/completions", json={"model": "m", "prompt": "x", "max_tokens": 2}).status_code == 500


def test_server_over_a_real_socket_and_model_loading_from_the_config(tmp_path):
    """``serve_async`` answers HTTP requests on a port; ``InferenceServer.create`` without a model loads the configured
    Hugging Face directory."""
    import asyncio
    import json
    import socket
    import urllib.request

    from levanter_b200.inference.openai import _load_model

    cfg_model = LlamaConfig(seq_len=64, hidden_dim=32, intermediate_dim=64, num_layers=1, num_heads=2, num_kv_heads=2)
    model = cfg_model.build(256, seed=0).eval()
    cfg_model.hf_checkpoint_converter().save_pretrained(model, str(tmp_path / "hf"), save_tokenizer=False)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cfg = InferenceServerConfig(model=cfg_model, hf_checkpoint=str(tmp_path / "hf"), host="127.0.0.1", port=port, batch_timeout=0.02,
                                service=InferenceEngineConfig(max_seqs=2, page_size=8, max_pages_per_seq=8, compute_dtype=torch.float32, max_rounds=2))
    loaded = _load_model(cfg, CharTokenizer())
    for (n, p), (_, q) in zip(model.named_parameters(), loaded.named_parameters()):
        assert torch.equal(p, q.float()), n
    srv = InferenceServer.create(cfg, model=loaded, tokenizer=CharTokenizer())

    async def scenario():
        task = asyncio.create_task(srv.serve_async())
        loop = asyncio.get_running_loop()

        def call():
            for _ in range(100):
                try:
                    with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                        health = json.loads(r.read())
                    break
                except OSError:
                    import time

                    time.sleep(0.05)
            req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", method="POST", headers={"Content-Type": "application/json"},
                                         data=json.dumps({"model": "m", "prompt": "hi", "max_tokens": 3, "temperature": 0.0}).encode())
            with urllib.request.urlopen(req, timeout=30) as r:
                return health, json.loads(r.read())

        health, body = await loop.run_in_executor(None, call)
        srv.shutdown()
        await asyncio.wait_for(task, 30)
        return health, body

    health, body = asyncio.run(scenario())
    assert health["status"] == "healthy" and body["object"] == "text_completion" and 1 <= body["usage"]["completion_tokens"] <= 3
