import json
import os
import time
import urllib.error
import urllib.request

import pytest

from archlab_b200.services import chat, reporting, rewards, storage, tracking


class _Client:
    def __init__(self):
        self.rows = []

    def log_metrics(self, run, step, values):
        self.rows.append((run, step, values))


def test_ledger_sync_is_exactly_once_and_skips_torn_tail(tmp_path):
    ledger = tmp_path / "metrics.jsonl"
    ledger.write_text('{"step": 1, "loss": 2.0}\n{"step": 2, "loss": 1.5, "ok": true, "bad": NaN}\n{"step": 3, "lo')
    c = _Client()
    s = tracking.LedgerSync(c, tmp_path / "state.json")
    assert s.sync("run", ledger) == 2 and c.rows[1][2] == {"loss": 1.5}
    with open(ledger, "a") as f:
        f.write('ss": 1.0}\n')
    s2 = tracking.LedgerSync(c, tmp_path / "state.json")           # restart: cursor persisted
    assert s2.sync("run", ledger) == 1 and [r[1] for r in c.rows] == [1, 2, 3]
    assert s2.sync("run", ledger) == 0


def test_single_writer_lock_and_process_status(tmp_path):
    lock = tmp_path / "lock"
    with tracking.SingleWriterLock(lock):
        with pytest.raises(RuntimeError):
            tracking.SingleWriterLock(lock).__enter__()
    lock.write_text("999999999")                                   # stale owner
    with tracking.SingleWriterLock(lock):
        pass
    pid, hb = tmp_path / "pid", tmp_path / "hb"
    pid.write_text(str(os.getpid()))
    hb.write_text("x")
    assert tracking.process_status(pid, hb)["state"] == "RUNNING"
    assert tracking.process_status(pid, hb, now=time.time() + 1000)["state"] == "STALLED"
    pid.write_text("999999999")
    assert tracking.process_status(pid, hb)["state"] == "EXITED"


def test_offload_verifies_and_retention_keeps_newest_complete(tmp_path):
    src = tmp_path / "a.bin"
    src.write_bytes(b"payload")
    j = storage.OffloadJournal(tmp_path / "j.sqlite")
    r = storage.transfer(src, tmp_path / "dst" / "a.bin", j)
    assert r["state"] == "verified" and storage.transfer(src, tmp_path / "dst" / "a.bin", j)["state"] == "already-verified"
    with pytest.raises(ValueError):
        storage.transfer(src, tmp_path / "dst" / "b.bin", j, expected_sha="0" * 64)
    with pytest.raises(ValueError):
        storage.confined(tmp_path, "../x")


def test_math_rewards_are_exact():
    ok = rewards.verify_math_answer("<think>1/3+1/6</think> The final answer is \\boxed{\\frac{1}{2}}", "0.5")
    assert ok.correct and ok.reward == 1.0 and ok.canonical_answer == "1/2"
    assert not rewards.verify_math_answer("\\boxed{0.333}", "1/3").correct
    assert rewards.verify_math_answer("Final answer: 1,234", "1234").correct
    assert rewards.verify_math_answer("50%", "1/2").correct
    assert rewards.verify_math_answer("\\boxed{1} and \\boxed{2}", "1").reason == "missing_or_unsupported_final_answer"
    assert rewards.verify_math_answer("<think>unfinished", "1").reason == "missing_or_unsupported_final_answer"
    assert rewards.verify_math_answer("2", "x+1").reason == "unsupported_reference"
    assert rewards.canonical_math_answer("2^10") == "1024" and rewards.canonical_math_answer("1/0") is None


def test_chat_front_validates_and_round_trips():
    models = {"ckpt-a": "normal"}
    good = {"model": "ckpt-a", "messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}], "max_tokens": 8}
    assert chat.validate_request(good, models)["messages"][0]["content"] == "hi"
    for bad in ({**good, "model": "x"}, {**good, "max_tokens": 9999}, {**good, "tools": [1]}, {**good, "temperature": 3},
                {**good, "messages": [{"role": "assistant", "content": "a"}]}):
        with pytest.raises(ValueError):
            chat.validate_request(bad, models)
    front = chat.ChatFront("127.0.0.1", 0, "tok", models, timeout=5)
    try:
        import threading

        def owner():
            t = front.next_ticket(timeout=5)
            t.finish("hello " + t.request["messages"][-1]["content"])

        threading.Thread(target=owner, daemon=True).start()
        req = urllib.request.Request(f"http://127.0.0.1:{front.port}/v1/chat/completions", data=json.dumps(good).encode(),
                                     headers={"Authorization": "Bearer tok", "Content-Type": "application/json"})
        out = json.loads(urllib.request.urlopen(req, timeout=5).read())
        assert out["choices"][0]["message"]["content"] == "hello hi"
        bad = urllib.request.Request(f"http://127.0.0.1:{front.port}/v1/chat/completions", data=b"{}",
                                     headers={"Authorization": "Bearer nope"})
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(bad, timeout=5)
        assert e.value.code == 401
        assert json.loads(urllib.request.urlopen(f"http://127.0.0.1:{front.port}/health", timeout=5).read())["phase"] == "serving"
    finally:
        front.close()


def test_reporting_pairs_by_seed(tmp_path):
    runs = {"baseline": {0: 1.00, 1: 1.10, 2: 0.90}, "kda": {0: 0.95, 1: 1.04, 2: 0.88}, "solo": {7: 1.0}}
    rows = reporting.paired_comparison(runs, "baseline")
    kda = next(r for r in rows if r["variant"] == "kda")
    assert kda["wins"] == 3 and abs(kda["delta_mean"] + 0.043333) < 1e-5 and len(rows) == 2
    m = tmp_path / "m.jsonl"
    m.write_text("".join(json.dumps({"step": i, "loss": 3.0 - 0.1 * i}) + "\n" for i in range(1, 21)))
    rows = reporting.read_metrics(m)
    assert abs(reporting.final_value(rows) - 1.45) < 1e-9 and len(reporting.learning_curve(rows, ema=0.9)) == 20
    assert reporting.markdown_table([{"a": 1, "b": 0.5}], ["a", "b"]).count("|") == 9


def test_chat_front_streams_server_sent_events():
    import threading

    models = {"ckpt-a": "normal"}
    body = {"model": "ckpt-a", "messages": [{"role": "user", "content": "count"}], "max_tokens": 8, "stream": True}
    front = chat.ChatFront("127.0.0.1", 0, "tok", models, timeout=5)
    try:
        def owner():
            t = front.next_ticket(timeout=5)
            for piece in ("one ", "two ", "three"):
                t.emit(piece)
            t.finish("one two three")
            t = front.next_ticket(timeout=5)                      # a loop that never emits still streams its text once
            t.finish("whole")
            t = front.next_ticket(timeout=5)
            t.emit("par")
            t.finish(error="device lost")

        threading.Thread(target=owner, daemon=True).start()

        def events():
            req = urllib.request.Request(f"http://127.0.0.1:{front.port}/v1/chat/completions", data=json.dumps(body).encode(),
                                         headers={"Authorization": "Bearer tok", "Content-Type": "application/json"})
            with urllib.request.urlopen(req, timeout=5) as resp:
                assert resp.headers["Content-Type"] == "text/event-stream" and resp.headers["X-Accel-Buffering"] == "no"
                raw = resp.read().decode()
            return [line[len("data: "):] for line in raw.split("\n\n") if line.startswith("data: ")]

        first = events()
        assert first[-1] == "[DONE]"
        chunks = [json.loads(e) for e in first[:-1]]
        assert chunks[0]["choices"][0]["delta"] == {"role": "assistant"} and chunks[0]["object"] == "chat.completion.chunk"
        assert [c["choices"][0]["delta"].get("content") for c in chunks[1:-1]] == ["one ", "two ", "three"]
        assert chunks[-1]["choices"][0]["finish_reason"] == "stop" and len({c["id"] for c in chunks}) == 1
        second = [json.loads(e) for e in events()[:-1]]
        assert [c["choices"][0]["delta"].get("content") for c in second[1:-1]] == ["whole"]
        third = events()
        assert json.loads(third[-2]) == {"error": {"message": "device lost"}} and third[-1] == "[DONE]"
    finally:
        front.close()
