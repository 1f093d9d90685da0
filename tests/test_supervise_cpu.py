"""Supervisor policy: resume planning, switch at the next checkpoint, waiting for GPUs, giving up."""
import json

from archlab_b200.train import supervise as sv


class FakeOps:
    def __init__(self):
        self.alive, self.free, self.started, self.stops = False, True, [], 0

    def trainer_alive(self):
        return self.alive

    def gpus_free(self):
        return self.free

    def start(self, launch, resume_from):
        self.started.append((launch, resume_from))

    def request_stop_after_checkpoint(self):
        self.stops += 1


def _spec(tmp_path, **kw):
    base = tmp_path / "base.yaml"
    base.write_text("a: 1\n")
    ck = tmp_path / "ckpt"
    ck.mkdir(exist_ok=True)
    return {"arm": "A", "base": str(base), "dir": str(tmp_path / "arm"), "checkpoints": str(ck), "data": "snap1", "source": "src1",
            "total_steps": 100, **kw}


def test_fresh_then_full_resume_and_switch(tmp_path):
    spec, ops = _spec(tmp_path), FakeOps()
    s = sv.Supervisor(spec, ops)
    v = s.tick()
    assert v.action == "launched" and v.detail["mode"] == "fresh" and v.detail["seed"] == 1000 and v.detail["resume_from"] is None
    ops.alive = True
    assert s.tick().action == "idle"
    (tmp_path / "ckpt" / "latest_checkpointed_iteration.txt").write_text("20\n")
    ops.alive = False
    v = s.tick()
    assert v.action == "launched" and v.detail["mode"] == "full" and v.detail["seed"] == 1000 and v.detail["resume_from"].endswith("global_step_20")
    ops.alive = True
    spec["data"] = "snap2"                                     # new data: stop at the next checkpoint, once
    assert s.tick().action == "switch_requested" and s.tick().action == "switch_requested" and ops.stops == 1
    (tmp_path / "ckpt" / "latest_checkpointed_iteration.txt").write_text("30\n")
    ops.alive = False
    v = s.tick()
    assert v.detail["mode"] == "fresh" and v.detail["seed"] == 1030
    rows = [json.loads(l) for l in open(tmp_path / "arm" / "LAUNCHES.jsonl")]
    assert [r["step"] for r in rows] == [0, 20, 30]


def test_waits_gives_up_and_finishes(tmp_path):
    spec, ops = _spec(tmp_path), FakeOps()
    s = sv.Supervisor(spec, ops)
    ops.free = False
    assert s.tick().action == "waiting_for_gpus" and not ops.started
    ops.free = True
    for _ in range(3):
        assert s.tick().action == "launched"                  # trainer dies each time without a checkpoint
    assert s.tick().action == "gave_up"
    (tmp_path / "ckpt" / "latest_checkpointed_iteration.txt").write_text("100\n")
    assert s.run(period_seconds=0, sleep=lambda _: None).action == "done"


def test_rotate_log(tmp_path):
    log = tmp_path / "train.log"
    assert sv.rotate_log(log) is None
    log.write_text("x")
    a = sv.rotate_log(log)
    log.write_text("y")
    b = sv.rotate_log(log)
    assert a != b and a.exists() and b.exists() and not log.exists()
