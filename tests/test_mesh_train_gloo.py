"""The mesh trainer steps on gloo ranks under tp x pp, tp x cp and dp x ep layouts; the loss goes down."""
import json
import os
import socket

import pytest
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, argv, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    from archlab_b200.train import mesh_train

    losses = mesh_train.train(mesh_train.parse_args(argv))
    out[rank] = losses


def _run(world, argv):
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), argv, out), nprocs=world, join=True)
        return dict(out)


def test_mesh_axes():
    from archlab_b200.train.mesh_train import build_mesh

    m = build_mesh(5, 8, 2, 2, 1)
    assert (m.tp_i, m.cp_i, m.dp_i, m.pp_i) == (1, 0, 0, 1) and m.dp == 2
    assert m.axis_ranks("tp") == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert [4, 6] in m.axis_ranks("dp") and [1, 5] in m.axis_ranks("pp")
    with pytest.raises(ValueError):
        build_mesh(0, 6, 4, 1, 1)


@pytest.mark.parametrize("world,extra", [
    (4, ["--model=qwen35_tiny", "--tp=2", "--pp=2", "--sequence-parallel"]),
    (4, ["--model=qwen35_tiny_dense", "--tp=2", "--cp=2", "--sequence-parallel"]),
    (2, ["--model=v41_tiny", "--ep=2"]),
    (4, ["--model=qwen35_tiny", "--tp=2", "--sequence-parallel"]),          # tp2 x dp2 with ZeRO-sharded optimizer state
])
def test_mesh_train_steps(tmp_path, world, extra):
    argv = extra + ["--seq-len=32", "--global-batch=4", "--steps=6", "--lr=3e-3", f"--run-dir={tmp_path}"]
    out = _run(world, argv)
    ref = out[0]
    assert all(abs(a - b) < 1e-5 for r in out.values() for a, b in zip(r, ref))      # every rank reports the same loss
    assert ref[-1] < ref[0]
    rows = [json.loads(l) for l in open(tmp_path / "metrics_rank0.jsonl")]
    assert len(rows) == 6 and rows[-1]["grad_norm"] > 0


def test_zero_adamw_matches_torch_adamw():
    import torch

    from archlab_b200.optim.zero import ZeroAdamW

    torch.manual_seed(0)
    a = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.LayerNorm(5), torch.nn.Linear(5, 3))
    b = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.LayerNorm(5), torch.nn.Linear(5, 3))
    b.load_state_dict(a.state_dict())
    decay = [p for p in b.parameters() if p.dim() >= 2]
    rest = [p for p in b.parameters() if p.dim() < 2]
    ref = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.0}], lr=1e-2, betas=(0.9, 0.95))
    opt = ZeroAdamW(a.parameters(), lr=1e-2, weight_decay=0.1)
    opt.zero_grad()
    for i in range(4):
        x = torch.randn(7, 6)
        a(x).pow(2).sum().backward()
        opt.reduce_gradients()
        opt.step()
        ref.zero_grad()
        b(x).pow(2).sum().backward()
        ref.step()
    for p, q in zip(a.parameters(), b.parameters()):
        assert torch.allclose(p, q, atol=1e-5, rtol=1e-4)


def test_resume_reproduces_the_uninterrupted_run_and_contract_is_enforced(tmp_path, monkeypatch):
    from archlab_b200.train import mesh_train

    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    base = ["--model=qwen35_tiny_dense", "--seq-len=32", "--global-batch=2", "--lr=3e-3", "--save-every=2"]
    full = mesh_train.train(mesh_train.parse_args(base + ["--steps=4", f"--run-dir={tmp_path / 'a'}"]))
    mesh_train.train(mesh_train.parse_args(base + ["--steps=2", f"--run-dir={tmp_path / 'b'}"]))
    # the contract pins everything but the step budget; a finished run directory is closed for good
    with pytest.raises(FileExistsError):
        mesh_train.train(mesh_train.parse_args(base + ["--steps=4", f"--run-dir={tmp_path / 'b'}"]))
    (tmp_path / "b" / "COMPLETE.json").unlink()
    with pytest.raises(ValueError):
        mesh_train.train(mesh_train.parse_args(base[:1] + ["--seq-len=64"] + base[2:] + ["--steps=4", "--resume", f"--run-dir={tmp_path / 'b'}"]))
    rest = mesh_train.train(mesh_train.parse_args(base + ["--steps=4", "--resume", f"--run-dir={tmp_path / 'b'}"]))
    assert len(rest) == 2 and rest == pytest.approx(full[2:], abs=1e-6)
    assert (tmp_path / "b" / "PARALLELISM.json").exists() and (tmp_path / "b" / "COMPLETE.json").exists()
    assert len(list((tmp_path / "b" / "contracts").glob("attempt-*.json"))) == 2


def test_factory_family_under_data_parallelism(tmp_path, monkeypatch):
    from archlab_b200.train import mesh_train

    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    from archlab_b200.models.factory import families

    fam = "nanochat" if "nanochat" in families() else families()[0]
    losses = mesh_train.train(mesh_train.parse_args([f"--model=factory:{fam}", "--seq-len=32", "--global-batch=2", "--micro-batch=2",
                                                     "--steps=3", f"--run-dir={tmp_path}"]))
    assert len(losses) == 3 and all(l == l for l in losses)


def test_stop_request_checkpoints_and_leaves_cleanly(tmp_path, monkeypatch):
    from archlab_b200.train import mesh_train

    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    run = tmp_path / "r"
    run.mkdir()

    def on_step(step, loss):
        if step == 1:
            (run / "STOP_REQUESTED.json").write_text("{}")

    argv = ["--model=qwen35_tiny_dense", "--seq-len=32", "--global-batch=2", "--steps=6", f"--run-dir={run}"]
    (run / "placeholder").write_text("")                          # a non-empty directory without a contract is a fresh run
    losses = mesh_train.train(mesh_train.parse_args(argv), on_step=on_step)
    assert len(losses) == 2
    assert json.loads((run / "STOPPED.json").read_text())["step"] == 2
    assert (run / "checkpoints" / "latest_checkpointed_iteration.txt").read_text().strip() == "2" and (run / "HEARTBEAT.json").exists()
    # a stopped run is not a completed one: no completion marker, the partial result says so
    assert not (run / "COMPLETE.json").exists() and not (run / "RUNNING.json").exists()
    assert json.loads((run / "result.json").read_text()) ["outcome"] == "stopped"
    # ... and it resumes where it stopped, reproducing the uninterrupted run
    full = mesh_train.train(mesh_train.parse_args(argv[:-1] + [f"--run-dir={tmp_path / 'full'}"]))
    rest = mesh_train.train(mesh_train.parse_args(argv + ["--resume"]))
    assert len(rest) == 4 and losses + rest == pytest.approx(full, abs=1e-6)
    assert (run / "COMPLETE.json").exists() and not (run / "STOPPED.json").exists()
    assert json.loads((run / "result.json").read_text())["steps"] == 6


def test_fully_sharded_linears_follow_the_replicated_run(tmp_path):
    """The same data-parallel job with replicated weights and with row-sharded linears: equal loss curves."""
    from archlab_b200.models.factory import families

    fam = "nanochat" if "nanochat" in families() else families()[0]
    base = [f"--model=factory:{fam}", "--seq-len=32", "--global-batch=4", "--micro-batch=2", "--steps=4", "--lr=3e-3"]
    if fam == "nanochat":
        base += ["--n-layer=2", "--model-set=n_embd=128", "--model-set=n_head=2", "--model-set=n_kv_head=2",
                 "--model-set=vocab_size=512"]
    plain = _run(2, base + [f"--run-dir={tmp_path / 'plain'}"])
    shard = _run(2, base + ["--fsdp", "--fsdp-min-features=64", f"--run-dir={tmp_path / 'fsdp'}"])
    assert all(abs(a - b) < 2e-3 * abs(a) for a, b in zip(plain[0], shard[0])), (plain[0], shard[0])
    assert shard[0][-1] < shard[0][0]
    norms = [[json.loads(l)["grad_norm"] for l in open(tmp_path / d / "metrics_rank0.jsonl")] for d in ("plain", "fsdp")]
    assert all(abs(a - b) < 2e-2 * a for a, b in zip(*norms)), norms        # same gradient scale, not only the same direction
    assert all(abs(a - b) < 1e-6 for a, b in zip(shard[0], shard[1]))


def test_hang_dump_writes_the_stacks_of_a_slow_step(tmp_path, capfd):
    """A step slower than --hang-dump-seconds leaves the Python stack of every thread on stderr."""
    import time

    from archlab_b200.train import mesh_train

    def slow(step, loss):
        if step == 0:
            time.sleep(1.6)

    args = mesh_train.parse_args(["--model=qwen35_tiny", "--seq-len=32", "--global-batch=2", "--steps=2", f"--run-dir={tmp_path}",
                                  "--hang-dump-seconds=0.5"])
    # the hook runs inside the step, so the armed dump fires while it sleeps
    mesh_train.train(args, on_step=slow)
    err = capfd.readouterr().err
    assert "Timeout (0:00:00.5" in err and "most recent call first" in err and "slow" in err
