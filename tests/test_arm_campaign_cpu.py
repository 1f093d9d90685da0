"""Sequential A/B/C campaign: matched probes are a precondition, arms run one after another, failure ends the campaign."""
import json
import sys

import pytest

from archlab_b200.train.arm_campaign import ArmCampaign, source_hashes, validate_probes

CONTRACT = {"runtime": "b200", "topology": {"dp": 8}, "seed": 1, "global_batch": 512, "micro_batch": 4, "manifest_sha256": "m" * 64,
            "train_prefixes": ["t0"], "heldout_prefixes": ["h0"], "eval_sequences": 64}


def probe(root, arm, sources, **edit):
    d = root / f"probe-{arm}"
    d.mkdir(parents=True)
    contract = {**CONTRACT, "arm": arm, "mode": "probe", "source_sha256": sources, **edit.get("contract", {})}
    (d / "RUN_CONTRACT.json").write_text(json.dumps(contract))
    (d / "PROBE_COMPLETE.json").write_text(json.dumps({"all_model_weights_bitwise_restored": True, "scheduler_restored": True,
                                                       "optimizer_tensors_bitwise_restored": edit.get("restored", True)}))
    (d / "INITIALIZATION.json").write_text(json.dumps({"common_parameter_sha256": edit.get("init", "i" * 64)}))
    rows = [{"event": "train", "first_microbatches_sha256": f"b{k}" + edit.get("order", "")} for k in range(3)] + [{"event": "eval", "heldout_tokens_sha256": "h"}]
    (d / "metrics.jsonl").write_text("".join(json.dumps(r) + "\n" for r in rows))
    return d


def sources_dir(tmp_path):
    src = tmp_path / "src"
    src.mkdir()
    (src / "model.py").write_text("x = 1\n")
    return src


def test_probe_gates(tmp_path):
    src = sources_dir(tmp_path)
    hashes = source_hashes(src)
    good = {a: probe(tmp_path / "ok", a, hashes) for a in "ABC"}
    assert validate_probes(good, hashes)["data_order"] == ["b0", "b1", "b2"]
    for name, edit, message in (("r", {"restored": False}, "restoration gate"), ("i", {"init": "j" * 64}, "initialisation mismatch"),
                                ("o", {"order": "x"}, "data-order mismatch"), ("c", {"contract": {"seed": 2}}, "contracts differ"),
                                ("s", {"contract": {"source_sha256": {"model.py": "0" * 64}}}, "exact sources"), ("m", {"contract": {"mode": "train"}}, "wrong probe evidence")):
        probes = {"A": probe(tmp_path / name, "A", hashes), "B": probe(tmp_path / name, "B", hashes, **edit)}
        with pytest.raises(ValueError, match=message):
            validate_probes(probes, hashes)


SCRIPT = "import json, sys, pathlib; d = pathlib.Path(sys.argv[1]); d.mkdir(parents=True); arm = d.name\n" \
         "if arm == sys.argv[2]: raise SystemExit(5)\n" \
         "(d / 'TRAINING_COMPLETE.json').write_text(json.dumps({'consumed_tokens': int(sys.argv[3])}))\n"


def campaign(tmp_path, name, fail="none", tokens=1000, reported=1000):
    src = tmp_path / "src" if (tmp_path / "src").exists() else sources_dir(tmp_path)
    hashes = source_hashes(src)
    probes = {a: probe(tmp_path / f"probes-{name}", a, hashes) for a in "ABC"}
    c = ArmCampaign(tmp_path / name, src, lambda arm, run_dir: [sys.executable, "-c", SCRIPT, str(run_dir), fail, str(reported)], expected_tokens=tokens,
                    poll_seconds=0.05)
    return c, probes


def test_arms_run_in_order_and_failures_end_the_campaign(tmp_path):
    c, probes = campaign(tmp_path, "ok")
    state = c.run(probes, install_signal_handlers=False)
    assert state["status"] == "complete" and state["arms"] == {"A": "complete", "B": "complete", "C": "complete"}
    with pytest.raises(ValueError, match="fresh-only"):
        c.run(probes, install_signal_handlers=False)
    c2, probes = campaign(tmp_path, "fail", fail="B")
    state = c2.run(probes, install_signal_handlers=False)
    assert state["status"] == "failed" and state["arms"] == {"A": "complete", "B": "failed", "C": "queued"} and state["exit_code"] == 5
    c3, probes = campaign(tmp_path, "short", reported=999)
    with pytest.raises(RuntimeError, match="incorrect completion token count"):
        c3.run(probes, install_signal_handlers=False)
    assert json.loads((tmp_path / "short" / "CAMPAIGN.json").read_text())["status"] == "failed" and (tmp_path / "short" / "FAILURE.json").exists()
    c4, probes = campaign(tmp_path, "stopped")
    c4.request_stop()
    state = c4.run(probes, install_signal_handlers=False)
    assert state["status"] == "stopped" and set(state["arms"].values()) == {"queued"}
