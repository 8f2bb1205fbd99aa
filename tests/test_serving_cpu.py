"""Continuous batching over the paged cache: every request gets the tokens it would get alone."""
import threading

import pytest
import torch

from ferrotorch_b200.models.generation import GenerationConfig, generate
from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
from ferrotorch_b200.models.serving import ContinuousBatcher, Request, RequestState, SamplingParams
from ferrotorch_b200.nn.paged import OutOfPages, PagedKVCache


@pytest.fixture(scope="module")
def served():
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=160, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=128)
    model = LlamaForCausalLM(cfg).float().eval()
    g = torch.Generator().manual_seed(3)
    lens, news = [5, 23, 9, 40, 3, 17, 31, 12], [12, 6, 20, 5, 16, 9, 7, 14]
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    alone = [generate(model, torch.tensor([p]), GenerationConfig.greedy(n))[0, len(p):].tolist() for p, n in zip(prompts, news)]
    return model, prompts, news, alone


@pytest.mark.parametrize("blocks,chunk,budget", [(64, 512, 2048), (12, 16, 2048), (9, 8, 11)], ids=["roomy", "tight", "starved"])
def test_batched_requests_get_the_tokens_of_a_run_alone(served, blocks, chunk, budget):
    model, prompts, news, alone = served
    b = ContinuousBatcher(model, num_blocks=blocks, block_size=8, max_running=4, max_seq_len=128, prefill_chunk=chunk,
                          max_tokens_per_step=budget, watermark=0.0)
    reqs = [b.submit(p, n) for p, n in zip(prompts, news)]
    stats = b.run()
    assert [r.output for r in reqs] == alone
    assert all(r.state is RequestState.FINISHED and r.finish_reason == "length" for r in reqs)
    assert b.manager.free_pages == blocks and b.manager.num_sequences() == 0 and not b.has_work()
    assert stats.peak_pages <= blocks and stats.peak_running <= 4 and max(stats.batch_tokens) <= budget
    assert stats.finished == len(reqs) and stats.decode_tokens + stats.prefill_tokens == sum(stats.batch_tokens)
    if blocks == 64:
        assert stats.preemptions == 0
        assert stats.steps < sum(news)                    # the requests shared their steps
        assert stats.prefill_tokens == sum(len(p) for p in prompts)
    else:                                                 # 4 sequences of up to 45 tokens do not fit into 9 or 12 pages of 8
        assert stats.preemptions > 0 and sum(r.preemptions for r in reqs) == stats.preemptions
        assert reqs[0].preemptions == 0                   # the oldest request is never the one that gives way
    assert all(0 <= r.submit_step <= r.first_token_step <= r.finish_step for r in reqs)


def test_a_sampled_request_does_not_depend_on_its_neighbours(served):
    model, prompts, news, _ = served
    sp = SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=11, repetition_penalty=1.1)

    def run(crowd):
        b = ContinuousBatcher(model, num_blocks=12 if crowd else 32, block_size=8, max_running=4, max_seq_len=128, watermark=0.0)
        others = [b.submit(p, n, sampling=SamplingParams(temperature=1.0, seed=i)) for i, (p, n) in enumerate(zip(prompts[2:6], news[2:6]))] if crowd else []
        r = b.submit(Request(prompts[1], 15, sampling=SamplingParams(**vars(sp))))
        b.run()
        return r.output, others

    solo, _ = run(False)
    crowded, others = run(True)
    assert solo == crowded and len(solo) == 15
    assert all(len(o.output) == n for o, n in zip(others, news[2:6]))
    # greedy with a repetition penalty goes through the host path and differs from plain greedy somewhere
    b = ContinuousBatcher(model, num_blocks=32, block_size=8, max_seq_len=128)
    a = b.submit(prompts[0], 12, sampling=SamplingParams(repetition_penalty=5.0))
    b.run()
    assert len(a.output) == 12 and len(set(a.output)) >= 6


def test_stop_ids_callbacks_cancellation_and_argument_checks(served):
    model, prompts, news, alone = served
    b = ContinuousBatcher(model, num_blocks=32, block_size=8, max_running=3, max_seq_len=128)
    stop_tok = alone[2][4]
    first = alone[2].index(stop_tok)
    seen = []
    r_stop = b.submit(prompts[2], 20, stop_ids=(stop_tok,))
    r_cb = b.submit(prompts[0], 12, on_token=lambda t: seen.append(t) or len(seen) < 3)
    r_cancel = b.submit(prompts[3], 5)
    r_late = b.submit(prompts[4], 16)                       # waits for a slot
    b.step()
    b.cancel(r_cancel)
    b.cancel(r_late)
    b.run()
    assert r_stop.output == alone[2][:first + 1] and r_stop.finish_reason == "stop"
    assert r_cb.output == alone[0][:3] == seen and r_cb.finish_reason == "stop"
    assert r_cancel.finish_reason == "cancelled" and r_late.finish_reason == "cancelled" and r_late.output == []
    assert b.manager.free_pages == 32
    with pytest.raises(ValueError):
        b.submit([], 4)
    with pytest.raises(ValueError):
        b.submit(prompts[0], 0)
    with pytest.raises(ValueError):
        b.submit(prompts[3], 100)                           # beyond max_seq_len
    with pytest.raises(ValueError):
        b.submit(prompts[0], 4, sampling=SamplingParams(top_p=0.0))
    small = ContinuousBatcher(model, num_blocks=2, block_size=8, max_seq_len=128)
    with pytest.raises(OutOfPages):
        small.submit(prompts[3], 5)                         # 45 tokens need 6 pages
    assert small.generate([prompts[4]], 8) == [alone[4][:8]]


def test_serving_loop_on_its_own_thread_takes_requests_from_others(served):
    model, prompts, news, alone = served
    b = ContinuousBatcher(model, num_blocks=24, block_size=8, max_running=4, max_seq_len=128)
    stop = threading.Event()
    loop = threading.Thread(target=b.serve_forever, args=(stop,))
    loop.start()
    try:
        got = {}

        def client(i):
            got[i] = b.submit(prompts[i], news[i]).result(timeout=120)

        clients = [threading.Thread(target=client, args=(i,)) for i in range(6)]
        [c.start() for c in clients]
        [c.join(120) for c in clients]
    finally:
        stop.set()
        loop.join(120)
    assert not loop.is_alive() and got == {i: alone[i] for i in range(6)}


def test_paged_decode_reads_the_sequences_it_is_given():
    torch.manual_seed(1)
    c = PagedKVCache(1, 2, 16, num_blocks=12, max_seqs=4, max_seq_len=32, block_size=4, device="cpu", dtype=torch.float32)
    lens = {0: 5, 2: 9, 3: 3}
    kv = {}
    for s, n in lens.items():
        c.reserve(s, n)
        k, v = torch.randn(n, 2, 16), torch.randn(n, 2, 16)
        c.append(0, k, v, torch.arange(n, dtype=torch.int32), torch.full((n,), s, dtype=torch.int32))
        kv[s] = (k, v)
    q = torch.randn(3, 4, 16)
    order = torch.tensor([3, 0, 2], dtype=torch.int32)
    out = c.decode(0, q, torch.tensor([3, 5, 9], dtype=torch.int32), seq_ids=order)
    for b, s in enumerate(order.tolist()):
        k, v = kv[s]
        kk, vv = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
        p = torch.softmax(torch.einsum("hd,nhd->hn", q[b], kk) / 4.0, -1)
        assert torch.allclose(out[b], torch.einsum("hn,nhd->hd", p, vv), atol=1e-5)
    with pytest.raises(ValueError):
        c.append(0, torch.zeros(1, 2, 16), torch.zeros(1, 2, 16), torch.tensor([20], dtype=torch.int32), torch.tensor([0], dtype=torch.int32))


def test_prefix_caching_shares_the_pages_of_a_common_prompt(served):
    model, prompts, news, alone = served
    g = torch.Generator().manual_seed(9)
    system = torch.randint(0, 160, (37,), generator=g).tolist()
    tails = [torch.randint(0, 160, (n,), generator=g).tolist() for n in (6, 11, 3, 8, 14, 1)]
    full = [system + t for t in tails]
    want = [generate(model, torch.tensor([p]), GenerationConfig.greedy(8))[0, len(p):].tolist() for p in full]

    plain = ContinuousBatcher(model, num_blocks=40, block_size=8, max_running=2, max_seq_len=128, watermark=0.0)
    assert plain.generate(full, 8) == want
    b = ContinuousBatcher(model, num_blocks=40, block_size=8, max_running=2, max_seq_len=128, watermark=0.0, prefix_caching=True)
    assert b.generate(full, 8) == want
    # the first two requests start together and compute the system prompt; the other four adopt its four whole pages
    assert b.stats.prefix_hit_tokens == 4 * 32 and b.stats.prefill_tokens == plain.stats.prefill_tokens - 4 * 32
    assert b.stats.steps <= plain.stats.steps and b.prefix.hits >= 16
    pool = b.cache.pool
    assert b.manager.num_sequences() == 0 and pool.num_used == len(b.prefix) > 0
    assert all(pool.ref_count(p) == 1 for p in b.prefix._table.values())
    # the same prompt again: everything but its last partial page is adopted, the answer is the same
    again = b.submit(full[1], 8)
    b.run()
    assert again.output == want[1] and b.stats.prefix_hit_tokens == 4 * 32 + 40
    b.prefix.clear()
    assert pool.num_used == 0 and pool.num_free == 40

    # a pool so small that listed pages have to be evicted to make room, and sequences preempted after that
    tight = ContinuousBatcher(model, num_blocks=14, block_size=8, max_running=3, max_seq_len=128, watermark=0.0, prefix_caching=True)
    assert tight.generate(full + [prompts[i] for i in (0, 2, 4, 5)], 8) == want + [alone[i][:8] for i in (0, 2, 4, 5)]
    assert tight.prefix.evictions > 0 and tight.cache.pool.num_used == len(tight.prefix)
    tight.prefix.clear()
    assert tight.cache.pool.num_free == 14


def test_page_pool_counts_holders():
    from ferrotorch_b200.nn.paged import PagePool

    pool = PagePool(3)
    a = pool.allocate()
    assert pool.retain(a) == a and pool.ref_count(a) == 2
    pool.free(a)
    assert pool.num_used == 1
    pool.free(a)
    assert pool.num_used == 0 and pool.ref_count(a) == 0
    with pytest.raises(ValueError):
        pool.free(a)
    with pytest.raises(ValueError):
        pool.retain(a)
    c = PagedKVCache(1, 1, 4, num_blocks=4, max_seqs=2, max_seq_len=16, block_size=4, device="cpu", dtype=torch.float32)
    c.reserve(0, 8)
    c.adopt(1, c.pages_of(0), 8)
    assert c.len(1) == 8 and c.pool.num_used == 2
    c.free_sequence(0)
    assert c.pool.num_used == 2
    c.free_sequence(1)
    assert c.pool.num_used == 0
    with pytest.raises(ValueError):
        c.adopt(1, [0], 3)


def test_http_front_serves_concurrent_completions_streams_and_reports_metrics(served):
    import json
    import urllib.error
    import urllib.request

    from ferrotorch_b200.models.server import ServingApp

    model, prompts, news, alone = served
    b = ContinuousBatcher(model, num_blocks=24, block_size=8, max_running=4, max_seq_len=128, prefix_caching=True)
    app = ServingApp(b, encode=lambda s: [ord(c) % 160 for c in s], decode=lambda ids: "".join(chr(65 + i % 26) for i in ids)).start()
    base = "http://127.0.0.1:%d" % app.port

    def post(body, raw=False):
        req = urllib.request.Request(base + "/v1/completions", json.dumps(body).encode(), {"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as resp:
            data = resp.read()
        return data if raw else json.loads(data)

    try:
        got = {}
        ts = [threading.Thread(target=lambda i=i: got.__setitem__(i, post({"prompt": prompts[i], "max_tokens": news[i]}))) for i in range(6)]
        [t.start() for t in ts]
        [t.join(120) for t in ts]
        for i in range(6):
            c = got[i]["choices"][0]
            assert c["token_ids"] == alone[i] and c["finish_reason"] == "length"
            assert c["text"] == "".join(chr(65 + t % 26) for t in alone[i])
            assert got[i]["usage"] == {"prompt_tokens": len(prompts[i]), "completion_tokens": news[i], "total_tokens": len(prompts[i]) + news[i]}
        assert len({got[i]["id"] for i in got}) == 6

        events = [json.loads(line[6:]) for line in post({"prompt": prompts[2], "max_tokens": 20, "stream": True, "stop_token_ids": [alone[2][7]], "lookahead": 3},
                                                        raw=True).decode().split("\n\n") if line.startswith("data: {")]
        upto = alone[2].index(alone[2][7]) + 1
        assert [e["token_id"] for e in events[:-1]] == alone[2][:upto] and [e["index"] for e in events[:-1]] == list(range(upto))
        assert events[-1]["finish_reason"] == "stop" and events[-1]["completion_tokens"] == upto

        text = post({"prompt": "hello there", "max_tokens": 4, "temperature": 0.7, "seed": 3})
        again = post({"prompt": "hello there", "max_tokens": 4, "temperature": 0.7, "seed": 3})
        assert text["choices"][0]["token_ids"] == again["choices"][0]["token_ids"] and len(text["choices"][0]["text"]) == 4

        for bad in ({"max_tokens": 4}, {"prompt": [], "max_tokens": 4}, {"prompt": [1, -2]}, {"prompt": [1], "max_tokens": 0},
                    {"prompt": [1], "top_p": 0}, {"prompt": [1] * 100, "max_tokens": 100}):
            with pytest.raises(urllib.error.HTTPError) as e:
                post(bad)
            assert e.value.code == 400 and "error" in json.loads(e.value.read())
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(base + "/nothing", timeout=30)
        assert e.value.code == 404

        health = json.loads(urllib.request.urlopen(base + "/health", timeout=30).read())
        assert health == {"status": "ok", "running": 0, "waiting": 0}
        metrics = urllib.request.urlopen(base + "/metrics", timeout=30).read().decode()
        values = {l.split()[0]: int(l.split()[1]) for l in metrics.splitlines() if not l.startswith("#")}
        assert values["ferrotorch_serving_requests_finished_total"] == 9 and values["ferrotorch_serving_kv_pages_total"] == 24
        assert values["ferrotorch_serving_decode_tokens_total"] == b.stats.decode_tokens > 0
        assert values["ferrotorch_serving_prefix_hit_tokens_total"] >= 16      # the streamed and the repeated prompts were listed
    finally:
        app.shutdown()
    assert not app._loop.is_alive() and app.loop_error is None


def test_server_command_line_starts_a_tiny_model_and_stops(capsys):
    from ferrotorch_b200.models import server

    assert server.main(["--tiny", "--device", "cpu", "--port", "0", "--kv-pages", "16", "--serve-seconds", "0.2"]) == 0
    assert "serving on http://127.0.0.1:" in capsys.readouterr().out
    with pytest.raises(SystemExit):
        server.main([])


def test_a_request_can_carry_a_grammar_while_its_neighbours_run_free():
    import json

    from ferrotorch_b200.models.generation import GrammarLogitsProcessor
    from ferrotorch_b200.utils.text import JsonGrammar

    vocab = ["{", "}", '"a"', '"b"', ":", ",", "1", "2", "[", "]", "true", " ", "<eos>", "x", "y", "z"]
    cfg = LlamaConfig(vocab_size=len(vocab), hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                      num_attention_heads=2, num_key_value_heads=1, head_dim=16, max_position_embeddings=128)
    torch.manual_seed(3)
    model = LlamaForCausalLM(cfg).float().eval()
    eos = vocab.index("<eos>")
    g = JsonGrammar()
    b = ContinuousBatcher(model, num_blocks=32, block_size=8, max_running=8, max_seq_len=64)
    constrained = [b.submit(Request([0, 4, 6], 24, (eos,), SamplingParams(temperature=1.5, seed=s),
                                    logits_processor=GrammarLogitsProcessor(g, vocab, eos))) for s in range(4)]
    free = [b.submit(Request([0, 4, 6], 24, (eos,), SamplingParams(temperature=1.5, seed=s))) for s in range(4)]
    b.run()
    for r in constrained:
        text = "".join(vocab[t] for t in r.output if t != eos)
        assert g.accepts_prefix(text), text
        if r.finish_reason == "stop":
            json.loads(text)
    assert any(not g.accepts_prefix("".join(vocab[t] for t in r.output if t != eos)) for r in free)


def test_lookup_speculation_keeps_the_greedy_output_and_saves_steps(served):
    model, prompts, news, alone = served
    assert ContinuousBatcher._look_up([1, 2, 3, 9, 1, 2, 3], 3, 4) == [9, 1, 2, 3]
    assert ContinuousBatcher._look_up([5, 6, 7, 8, 6], 3, 2) == [7, 8] and ContinuousBatcher._look_up([1, 2, 3], 3, 4) == []
    # random weights make greedy decoding fall into a loop, which is what the look-up finds
    loop_prompt = prompts[0]
    want = generate(model, torch.tensor([loop_prompt]), GenerationConfig.greedy(60))[0, len(loop_prompt):].tolist()
    plain = ContinuousBatcher(model, num_blocks=32, block_size=8, max_seq_len=128)
    plain.submit(loop_prompt, 60)
    plain.run()
    for pool in (32, 11):
        b = ContinuousBatcher(model, num_blocks=pool, block_size=8, max_running=4, max_seq_len=128, watermark=0.0, prefix_caching=True)
        r = b.submit(Request(loop_prompt, 60, lookahead=5))
        others = [b.submit(Request(p, n, lookahead=3 if i % 2 else 0)) for i, (p, n) in enumerate(zip(prompts[1:5], news[1:5]))]
        stop_at = b.submit(Request(prompts[2], 20, (alone[2][9],), lookahead=4))
        b.run()
        assert r.output == want and [o.output for o in others] == alone[1:5]
        assert stop_at.output == alone[2][:alone[2].index(alone[2][9]) + 1] and stop_at.finish_reason == "stop"
        st = b.stats
        assert 0 < st.spec_accepted <= st.spec_proposed and st.decode_tokens + st.prefill_tokens == sum(st.batch_tokens)
        assert b.manager.num_sequences() == 0 and b.cache.pool.num_used == len(b.prefix)
    if len(set(want)) < 30:                                   # the output does loop: speculation must have paid
        solo = ContinuousBatcher(model, num_blocks=32, block_size=8, max_seq_len=128)
        solo.submit(Request(loop_prompt, 60, lookahead=5))
        solo.run()
        assert solo.stats.steps < plain.stats.steps
    # sampled requests ignore the option
    a = ContinuousBatcher(model, num_blocks=32, block_size=8, max_seq_len=128)
    x = a.submit(Request(prompts[1], 10, sampling=SamplingParams(temperature=0.9, seed=5), lookahead=4))
    a.run()
    assert a.stats.spec_proposed == 0 and len(x.output) == 10


def test_http_front_reports_a_failed_serving_loop(served):
    import json
    import urllib.error
    import urllib.request

    from ferrotorch_b200.models.server import ServingApp

    model, prompts, _, _ = served
    b = ContinuousBatcher(model, num_blocks=16, block_size=8, max_seq_len=128)

    def broken(runs):
        raise RuntimeError("injected on the host")

    b._forward = broken
    app = ServingApp(b).start()
    try:
        req = urllib.request.Request("http://127.0.0.1:%d/v1/completions" % app.port, json.dumps({"prompt": prompts[0], "max_tokens": 4}).encode())
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(req, timeout=60)
        assert e.value.code == 500 and "injected on the host" in json.loads(e.value.read())["error"]
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen("http://127.0.0.1:%d/health" % app.port, timeout=60)
        assert e.value.code == 500
    finally:
        app.shutdown()
    assert isinstance(app.loop_error, RuntimeError)
