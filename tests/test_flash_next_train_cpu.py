"""Native trainer entry of the Qwen3.8 family: run contract, resume refusals, probe hooks, bounded checkpoint staging."""
import json

import pytest
import torch

from archlab_b200.train import flash_next_train as T


def test_contract_is_written_once_and_resume_checks_what_matters(tmp_path):
    run = tmp_path / "run"
    base = ["--model-variant", "tiny", "--run-dir", str(run), "--seq-len", "32", "--global-batch", "2", "--contract-only"]
    assert T.main(base) == 0
    c = json.loads((run / "RUN_CONTRACT.json").read_text())
    assert c["training"]["loss_normalization"] == T.LOSS_NORMALIZATION and c["precision"]["precision"] == "bf16"
    assert c["optimizer"]["newton_schulz_steps"] == 8 and c["training"]["tokens_per_step"] == 64
    assert c["parameter_count"]["total"] > 0 and c["implementation_sha256"]["models/qwen38.py"]
    assert c["optimizer_partition"]["optimizers"]["muon"]["logical_matrices"] >= 1
    with pytest.raises(RuntimeError, match="already contains a contract"):
        T.main(base)
    assert T.main(base + ["--resume"]) == 0
    assert len(list((run / "contracts").glob("attempt-*.json"))) == 2 and (run / "LATEST_CONTRACT.json").exists()
    with pytest.raises(RuntimeError, match="precision recipe changed"):
        T.main(base + ["--resume", "--precision", "fp4"])
    with pytest.raises(RuntimeError, match="model geometry changed"):
        T.main(["--model-variant", "tiny", "--run-dir", str(run), "--seq-len", "64", "--global-batch", "2", "--contract-only", "--resume"])
    with pytest.raises(RuntimeError, match="lacks a RUN_CONTRACT"):
        T.main(["--model-variant", "tiny", "--run-dir", str(tmp_path / "other"), "--seq-len", "32", "--contract-only",
                "--load-dir", str(tmp_path / "nowhere" / "checkpoints")])
    for key, msg in (("loss_normalization", "loss normalization"), ("attention_grouping", "attention grouping")):
        changed = json.loads(json.dumps(c))
        changed["training"][key] = "something else"
        with pytest.raises(RuntimeError, match=msg):
            T.validate_resume(c, changed)


def test_probe_hooks_record_seen_and_nonfinite_gradients():
    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_gate = torch.nn.Linear(4, 4, bias=False)
            self.q_norm = torch.nn.LayerNorm(4)
            self.unused = torch.nn.Module()
            self.unused.k_norm = torch.nn.LayerNorm(4)

        def forward(self, x):
            return (self.q_norm(self.q_gate(x)) * torch.arange(4.0)).sum()      # a plain sum of LayerNorm outputs has no gradient

    m = M()
    rec = T.install_probe_hooks(m)
    assert set(rec) == {"q_gate.weight", "q_norm.weight", "unused.k_norm.weight"}
    m(torch.randn(3, 4)).backward()
    assert rec["q_gate.weight"]["seen"] and not rec["q_gate.weight"]["nonfinite"] and not rec["unused.k_norm.weight"]["seen"]
    (m.q_gate(torch.randn(2, 4)).sum() * float("inf")).backward()
    assert rec["q_gate.weight"]["nonfinite"]


def test_bounded_staging_serialises_the_local_ranks():
    from archlab_b200.train.mesh_train import staged_by_local_rank

    order, barriers = [], []
    for rank in range(3):                                  # the ranks of one host, simulated one after the other
        staged_by_local_rank(lambda r=rank: order.append(r), local_rank=rank, local_world=3, barrier=lambda: barriers.append(1))
    assert order == [0, 1, 2] and len(barriers) == 9       # each rank passes every turn's barrier, writes in its own
    with pytest.raises(RuntimeError):
        staged_by_local_rank(lambda: None, local_rank=3, local_world=3, barrier=lambda: None)
