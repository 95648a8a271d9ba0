"""Serving engine on CPU: tokens must equal the greedy full-recompute loop; scheduler and allocator logic."""
import pytest
import torch

from llm_systems_from_scratch_b200.models.transformer import TransformerLM
from llm_systems_from_scratch_b200.serving import PageAllocator, Request, Scheduler, ServingEngine, poisson_trace

CFG = dict(vocab_size=101, context_length=64, d_model=64, num_layers=2, num_heads=4, d_ff=136, rope_theta=10000.0)


def _greedy_reference(model, prompt, n):
    ids = torch.tensor([prompt])
    out = []
    for _ in range(n):
        nxt = int(model(ids)[0, -1].float().argmax())
        out.append(nxt)
        ids = torch.cat((ids, torch.tensor([[nxt]])), dim=1)
    return out


def test_engine_tokens_equal_full_recompute():
    torch.manual_seed(0)
    model = TransformerLM(**CFG).eval()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 101, (n,), generator=g).tolist() for n in (5, 17, 9, 30)]
    want = [_greedy_reference(model, p, 6) for p in prompts]
    eng = ServingEngine(model, page_size=4, max_batch=3, max_context=64)     # batch < requests: queueing happens
    got = eng.generate(prompts, 6)
    assert got == want
    assert eng.cache.allocator.free == eng.cache.num_pages                  # every page was returned
    assert eng.stats["decode_steps"] >= 5 and eng.stats["prefill_tokens"] == sum(map(len, prompts))


def test_eos_stops_a_request_early():
    torch.manual_seed(0)
    model = TransformerLM(**CFG).eval()
    prompt = [3, 1, 4, 1, 5]
    ref = _greedy_reference(model, prompt, 8)
    eos = ref[2]
    eng = ServingEngine(model, page_size=4, max_batch=2, max_context=64)
    out = eng.generate([prompt], 8, eos_token_id=eos)[0]
    assert out == ref[:ref.index(eos) + 1]


def test_allocator_and_scheduler_fcfs():
    a = PageAllocator(10)
    p = a.take(3)
    assert len(set(p)) == 3 and a.free == 7
    with pytest.raises(MemoryError):
        a.take(8)
    a.give(p)
    assert a.free == 10
    s = Scheduler(a, page_size=4, max_batch=2, max_prefill_tokens=20, max_context=40)
    reqs = [Request(0, [1] * 10, 6, 0.0), Request(1, [1] * 12, 4, 0.5), Request(2, [1] * 4, 4, 0.6)]
    for r in reqs:
        s.add(r)
    first = s.admit(0.1)
    assert [r.rid for r in first] == [0] and len(reqs[0].pages) == 4      # 16 tokens reserved -> 4 pages
    s.start(first)
    second = s.admit(1.0)
    assert [r.rid for r in second] == [1]                                  # batch limit 2: request 2 waits
    s.start(second)
    reqs[0].output = [7] * 6
    assert [r.rid for r in s.retire(2.0)] == [0] and a.free == 10 - 4
    assert [r.rid for r in s.admit(2.0)] == [2]
    with pytest.raises(ValueError):
        s.add(Request(9, [1] * 39, 5, 0.0))


def test_poisson_trace_statistics():
    tr = poisson_trace(2000, 20.0, (128, 2048), (64, 512), 50257, seed=0)
    gaps = [b.arrival - a.arrival for a, b in zip(tr, tr[1:])]
    assert abs(sum(gaps) / len(gaps) - 0.05) < 0.005
    assert min(len(r.prompt) for r in tr) >= 128 and max(len(r.prompt) for r in tr) <= 2048
    assert min(r.max_new_tokens for r in tr) >= 64 and max(r.max_new_tokens for r in tr) <= 512


def test_host_runtime_matches_python_paths():
    """C++ host runtime: window gather, page pool order, slot and block-table arithmetic against the Python code."""
    import numpy as np
    import pytest
    import torch
    from llm_systems_from_scratch_b200.serving.kv_cache import PageAllocator
    from llm_systems_from_scratch_b200.utils import host_runtime as hr
    if not hr.available():
        pytest.skip("no C++ compiler for the host runtime")
    rng = np.random.default_rng(0)
    tokens = rng.integers(0, 50000, size=1 << 18, dtype=np.uint32)
    starts = rng.integers(0, len(tokens) - 513, size=256, dtype=np.int64)
    out = torch.empty(256, 513, dtype=torch.int64)
    hr.gather_windows(tokens, starts, 513, out)
    want = tokens[np.arange(513)[None, :] + starts[:, None]].astype(np.int64)
    assert np.array_equal(out.numpy(), want)
    with pytest.raises(IndexError):
        hr.gather_windows(tokens, np.array([len(tokens) - 10], dtype=np.int64), 513, torch.empty(1, 513, dtype=torch.int64))
    a, b = PageAllocator(64, native=True), PageAllocator(64, native=False)
    held_a, held_b = [], []
    for step in range(200):
        if rng.random() < 0.6 and a.free >= 5:
            n = int(rng.integers(1, 6))
            held_a.append(a.take(n))
            held_b.append(b.take(n))
        elif held_a:
            i = int(rng.integers(0, len(held_a)))
            a.give(held_a.pop(i))
            b.give(held_b.pop(i))
        assert held_a == held_b and a.free == b.free
    with pytest.raises(MemoryError):
        a.take(a.free + 1)
    pages = [7, 3, 9]
    assert hr.slots(pages, 16, 14, 20) == [pages[t // 16] * 16 + t % 16 for t in range(14, 34)]
    table = hr.block_table([[1, 2, 3], [4], []], 4, pad=-1)
    assert table.tolist() == [[1, 2, 3, -1], [4, -1, -1, -1], [-1, -1, -1, -1]]


def test_generate_runs_through_the_paged_kv_engine():
    """``TransformerLM.generate`` on the fused engine (prefill + cached decode steps) returns the tokens of the
    reference-style loop that re-runs the whole context for every token; the stop token is not returned."""
    from llm_systems_from_scratch_b200.models.transformer import TransformerLM
    torch.manual_seed(0)
    cfg = dict(vocab_size=211, context_length=64, d_model=64, num_layers=2, num_heads=4, d_ff=136, rope_theta=10000.0)
    fused = TransformerLM(**cfg, use_custom_triton=True).eval()
    eager = TransformerLM(**cfg, use_custom_triton=False).eval()
    eager.load_state_dict(fused.canonical_state_dict())
    prompt = torch.randint(0, 211, (9,), generator=torch.Generator().manual_seed(3))
    want = eager.generate(prompt, 12, temperature=0)            # eager modules: the re-forward loop
    got = fused.generate(prompt, 12, temperature=0)             # fused engine: paged KV cache
    assert got.shape == (1, 12) and torch.equal(got, want)
    stop = int(want[0, 5])
    cut = fused.generate(prompt, 12, temperature=0, eos_token_id=stop)
    first = want[0].tolist().index(stop)
    assert cut[0].tolist() == want[0, :first].tolist()
    torch.manual_seed(1)
    sampled = fused.generate(prompt, 12, temperature=0.8, top_k=5)
    assert sampled.shape == (1, 12) and int(sampled.max()) < 211
    # beyond the context window the sliding re-forward loop still serves the call
    long = fused.generate(prompt, 64, temperature=0)
    assert long.shape == (1, 64)


def test_realtime_trace_and_requests_that_can_never_fit():
    """A small Poisson trace against the wall clock: every request is served, time to first token and latency are
    measured from its arrival, tokens equal the offline run.  A request that needs more pages than the cache holds is
    refused when it is submitted; one that fits the cache but not beside nothing at all is reported, not waited for."""
    torch.manual_seed(0)
    model = TransformerLM(**CFG).eval()
    trace = poisson_trace(12, 200.0, (4, 20), (3, 6), CFG["vocab_size"], seed=3)
    eng = ServingEngine(model, page_size=4, max_batch=4, max_context=64)
    res = eng.run(trace, realtime=True)
    assert res["requests"] == 12 and res["output_tokens"] == sum(r.max_new_tokens for r in trace)
    assert res["ttft_p50_s"] >= 0 and res["latency_p50_s"] >= res["ttft_p50_s"]
    assert all(r.t_first is not None and r.t_done >= r.t_first >= r.arrival for r in trace)
    again = poisson_trace(12, 200.0, (4, 20), (3, 6), CFG["vocab_size"], seed=3)
    eng2 = ServingEngine(model, page_size=4, max_batch=4, max_context=64)
    eng2.run(again, realtime=False)
    assert [r.output for r in again] == [r.output for r in trace]
    small = ServingEngine(model, num_pages=3, page_size=4, max_batch=2, max_context=64)
    with pytest.raises(ValueError):
        small.sched.add(Request(0, [1] * 10, 8, 0.0))          # 18 positions = 5 pages > 3


def test_context_splits_fill_the_waves_of_the_attention_launch():
    """``choose_splits`` is host arithmetic: for the 2048-wide model two CTAs fit on an SM (296 per wave on 148 SMs);
    the chosen split count never leaves less than 256 tokens per split at full context, and no other admissible count
    fills its last wave better."""
    from llm_systems_from_scratch_b200.ops.serving_ops import choose_splits
    resident = 148 * 2
    fill = lambda ctas: ctas / (-(-ctas // resident) * resident)
    for rows in (1, 3, 16, 32, 48, 64, 96, 128, 160, 192, 224, 256, 300):
        s = choose_splits(rows, 16, 2048)
        assert 1 <= s <= 8
        assert all(fill(rows * s) >= fill(rows * other) - 1e-9 for other in range(1, 9))
    assert choose_splits(128, 16, 2048) == 8          # 1024 CTAs = 3.46 waves of 296: 0.865 full, like 2, 4 and 6; ties go up
    assert choose_splits(48, 16, 2048) == 6           # 288 of 296
    assert choose_splits(5, 4, 256, head_dim=128) == 1    # a short context is not split
    assert choose_splits(64, 12, 1024, head_dim=64) <= 4


def test_online_server_serves_concurrent_requests_with_the_tokens_of_the_greedy_loop():
    """``EngineServer``: requests submitted from several threads while others are decoding get exactly the tokens of
    the per-request greedy recompute loop; a request that can never fit is refused to its caller only; every page is
    back in the pool afterwards."""
    import threading
    from llm_systems_from_scratch_b200.serving.server import EngineServer
    torch.manual_seed(0)
    model = TransformerLM(**CFG).eval()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 101, (n,), generator=g).tolist() for n in (5, 17, 9, 30, 3, 12, 21)]
    want = [_greedy_reference(model, p, 7) for p in prompts]
    eng = ServingEngine(model, page_size=4, max_batch=3, max_context=64)
    server = EngineServer(eng).start()
    try:
        got = [None] * len(prompts)

        def client(i):
            got[i] = server.generate(prompts[i], 7, timeout=120)

        threads = [threading.Thread(target=client, args=(i,)) for i in range(len(prompts))]
        for t in threads:
            t.start()
        for t in threads:
            t.join(180)
        assert [c.output_ids for c in got] == want
        assert all(c.ttft_s is not None and 0 <= c.ttft_s <= c.latency_s for c in got)
        with pytest.raises(Exception):
            server.generate(list(range(60)), 30, timeout=30)         # 90 tokens do not fit a context of 64
        assert server.generate(prompts[0], 7, timeout=60).output_ids == want[0]     # the loop is still serving
        s = server.stats()
        assert s["alive"] and s["completed"] == len(prompts) + 1 and s["running"] == 0
    finally:
        server.stop()
    assert eng.cache.allocator.free == eng.cache.num_pages


def test_http_front_end():
    from fastapi.testclient import TestClient
    from llm_systems_from_scratch_b200.serving.server import EngineServer, build_app
    torch.manual_seed(0)
    model = TransformerLM(**CFG).eval()
    eng = ServingEngine(model, page_size=4, max_batch=4, max_context=64)
    server = EngineServer(eng).start()
    try:
        client = TestClient(build_app(server, default_max_new_tokens=5))
        assert client.get("/health").json() == {"status": "ok"}
        prompt = [3, 1, 4, 1, 5, 9, 2, 6]
        r = client.post("/generate", json={"prompt_ids": prompt, "max_new_tokens": 6})
        assert r.status_code == 200
        body = r.json()
        assert body["output_ids"] == _greedy_reference(model, prompt, 6) and body["latency_ms"] >= body["ttft_ms"] >= 0
        assert len(client.post("/generate", json={"prompt_ids": prompt}).json()["output_ids"]) == 5
        assert client.post("/generate", json={"prompt": "text without a tokenizer"}).status_code == 422
        assert client.post("/generate", json={"prompt_ids": list(range(60)), "max_new_tokens": 30}).status_code == 400
        stats = client.get("/stats").json()
        assert stats["completed"] == 2 and stats["kv_pages"] == eng.cache.num_pages
    finally:
        server.stop()


def test_server_cancellation_frees_the_row_and_the_pages():
    """A cancelled request (a client that went away) resolves with what it has and ``cancelled=True``, whether it was
    still waiting or already decoding; its KV pages are back in the pool and the requests around it still get exactly
    the tokens of the greedy loop."""
    import time
    from llm_systems_from_scratch_b200.serving.server import EngineServer
    torch.manual_seed(0)
    model = TransformerLM(**CFG).eval()
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 101, (n,), generator=g).tolist() for n in (6, 11, 8)]
    want = [_greedy_reference(model, p, 20) for p in prompts]
    eng = ServingEngine(model, page_size=4, max_batch=2, max_context=64)
    server = EngineServer(eng).start()
    try:
        seen = []
        futs = [server.submit(prompts[0], 20),
                server.submit(prompts[1], 40, on_tokens=seen.extend),      # the one to cancel while it decodes
                server.submit(prompts[2], 20)]                             # waits: the batch holds two
        late = server.submit(prompts[0], 30)                               # cancelled while still waiting
        server.cancel(late.request_id)
        while len(seen) < 3:                                               # let the victim produce a few tokens
            time.sleep(0.001)
        server.cancel(futs[1].request_id)
        done = [f.result(120) for f in futs]
        gone = late.result(120)
        assert gone.cancelled and gone.output_ids == [] and gone.ttft_s is None
        assert done[1].cancelled and 3 <= len(done[1].output_ids) < 40
        assert done[1].output_ids == _greedy_reference(model, prompts[1], len(done[1].output_ids))
        assert not done[0].cancelled and done[0].output_ids == want[0] and done[2].output_ids == want[2]
        server.cancel(futs[0].request_id)                                  # finished already: ignored
        assert server.generate(prompts[1], 20, timeout=60).output_ids == want[1]
    finally:
        server.stop()
    assert eng.cache.allocator.free == eng.cache.num_pages


def test_server_back_pressure():
    """With ``max_waiting`` the server refuses what it cannot hold instead of queueing without bound (HTTP 503)."""
    from fastapi.testclient import TestClient
    from llm_systems_from_scratch_b200.serving.server import EngineServer, QueueFull, build_app
    torch.manual_seed(0)
    model = TransformerLM(**CFG).eval()
    server = EngineServer(ServingEngine(model, page_size=4, max_batch=2, max_context=64), max_waiting=0).start()
    try:
        with pytest.raises(QueueFull):
            server.submit([1, 2, 3], 4)
        r = TestClient(build_app(server)).post("/generate", json={"prompt_ids": [1, 2, 3], "max_new_tokens": 4})
        assert r.status_code == 503 and r.headers["retry-after"] == "1"
        server.max_waiting = 8
        assert len(server.generate([1, 2, 3], 4, timeout=60).output_ids) == 4
    finally:
        server.stop()


def test_http_streaming_and_metrics():
    """``"stream": true`` answers with server-sent events whose token batches concatenate to the greedy loop's output
    and end with the timings; ``/metrics`` exposes the counters in the Prometheus text format."""
    import json
    from fastapi.testclient import TestClient
    from llm_systems_from_scratch_b200.serving.server import EngineServer, build_app
    torch.manual_seed(0)
    model = TransformerLM(**CFG).eval()
    eng = ServingEngine(model, page_size=4, max_batch=4, max_context=64)
    server = EngineServer(eng).start()
    try:
        client = TestClient(build_app(server))
        prompt = [7, 3, 9, 1, 12, 40]
        want = _greedy_reference(model, prompt, 9)
        with client.stream("POST", "/generate", json={"prompt_ids": prompt, "max_new_tokens": 9, "stream": True}) as r:
            assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
            events = [json.loads(line[len("data: "):]) for line in r.iter_lines() if line.startswith("data: ")]
        assert events[-1].get("done") is True and events[-1]["latency_ms"] >= events[-1]["ttft_ms"] >= 0
        assert sum((e["output_ids"] for e in events[:-1]), []) == want
        assert len(events) > 2                                  # tokens arrived in more than one batch
        # callbacks straight on the server object
        seen = []
        done = server.submit(prompt, 5, on_tokens=seen.extend).result(60)
        assert seen == done.output_ids == want[:5]
        text = client.get("/metrics").text
        assert "llm_requests_completed_total 2" in text and f"llm_output_tokens_total {9 + 5}" in text
        assert 'llm_ttft_seconds{quantile="0.5"}' in text and "llm_kv_cache_occupancy 0" in text
    finally:
        server.stop()
    assert eng.cache.allocator.free == eng.cache.num_pages


def test_http_front_end_with_text_prompts():
    """With a tokenizer the app takes text and answers with text; the ids are those of the greedy loop on the encoded
    prompt."""
    import os
    from fastapi.testclient import TestClient
    from llm_systems_from_scratch_b200.serving.server import EngineServer, build_app
    from llm_systems_from_scratch_b200.tokenizer.bpe import Tokenizer
    data = os.path.join(os.path.dirname(__file__), "data")
    tok = Tokenizer.from_files(os.path.join(data, "vocab.json"), os.path.join(data, "merges.json"),
                               special_tokens=["<|endoftext|>"])
    torch.manual_seed(0)
    model = TransformerLM(**dict(CFG, vocab_size=len(tok.id_to_bytes))).eval()
    server = EngineServer(ServingEngine(model, page_size=4, max_batch=4, max_context=64)).start()
    try:
        client = TestClient(build_app(server, tok, default_max_new_tokens=6))
        body = client.post("/generate", json={"prompt": "the cat"}).json()
        assert body["output_ids"] == _greedy_reference(model, tok.encode("the cat"), 6)
        assert body["text"] == tok.decode(body["output_ids"])
    finally:
        server.stop()
