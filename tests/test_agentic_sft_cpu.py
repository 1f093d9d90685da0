"""Agent-trajectory SFT data: tool-turn contract, prefix-stable assistant masks, recorded-token rows, splits, packing."""
import json

import numpy as np
import pytest

from archlab_b200.data import agentic_sft as ag

EOS = 9


def call(cid, **args):
    return {"id": cid, "type": "function", "function": {"name": "bash", "arguments": json.dumps(args)}}


def episode():
    return [{"role": "system", "content": "source prompt (dropped)"}, {"role": "user", "content": "fix the bug"},
            {"role": "assistant", "content": "looking", "tool_calls": [call("c1", command="ls", timeout=30)]},
            {"role": "tool", "tool_call_id": "c1", "content": [{"type": "text", "text": "a.py"}]},
            {"role": "assistant", "content": "done"}]


def test_tool_turns_follow_the_runtime_contract():
    out = ag.normalize_tool_messages(episode(), system="deployed agent prompt")
    assert out[0] == {"role": "system", "content": "deployed agent prompt"} and out[3]["content"] == "a.py"
    assert json.loads(out[2]["tool_calls"][0]["function"]["arguments"]) == {"command": "ls", "timeout": 30}

    def broken(edit):
        e = episode()
        edit(e)
        return e
    cases = {
        "non-bash": lambda e: e[2]["tool_calls"][0]["function"].update(name="python"),
        "arguments differ": lambda e: e[2]["tool_calls"][0]["function"].update(arguments=json.dumps({"command": "ls", "cwd": "/"})),
        "outside the runtime contract": lambda e: e[2]["tool_calls"][0]["function"].update(arguments=json.dumps({"command": "ls", "timeout": 900})),
        "no matching call": lambda e: e[3].update(tool_call_id="zz"),
        "one tool call per": lambda e: e[2]["tool_calls"].append(call("c2", command="pwd")),
        "finish with an idle": lambda e: e.pop(),
        "precedes its tool observations": lambda e: e.insert(3, {"role": "assistant", "content": "impatient"}),
    }
    for message, edit in cases.items():
        with pytest.raises(ValueError, match=message.replace("non-bash", "other than bash")):
            ag.normalize_tool_messages(broken(edit), system="s")


def render(history):
    """Toy template: [role id, *bytes, EOS-if-assistant]."""
    ids = []
    for m in history:
        ids += [{"system": 1, "user": 2, "assistant": 3, "tool": 4}[m["role"]]] + [10 + b for b in m["content"].encode()]
        if m["role"] == "assistant":
            ids.append(EOS)
    return ids


def test_assistant_spans_are_masked_through_their_single_eos():
    msgs = ag.normalize_tool_messages(episode(), system="s")
    row = ag.encode_assistant_targets(render, msgs, eos_token_id=EOS, max_length=200)
    ids, mask = row["input_ids"], row["loss_mask"]
    assert sum(mask) == (1 + len("looking") + 1) + (1 + len("done") + 1) and mask[0] == 0
    assert all(ids[j] == EOS for j in range(len(ids)) if mask[j] and (j + 1 == len(ids) or not mask[j + 1]))
    with pytest.raises(ValueError, match="exceeds the context"):
        ag.encode_assistant_targets(render, msgs, eos_token_id=EOS, max_length=10)

    def unstable(history):                                                # re-serialises earlier assistant turns differently
        ids = render(history)
        return ids if len(history) < 5 else [7] + ids
    with pytest.raises(ValueError, match="prefix-stable"):
        ag.encode_assistant_targets(unstable, msgs, eos_token_id=EOS, max_length=200)
    with pytest.raises(ValueError, match="exactly one EOS"):
        ag.encode_assistant_targets(render, msgs, eos_token_id=8, max_length=200)


def _npz(path, prompt, response, mask, spans):
    np.savez(path, traj0_prompt_ids=np.array(prompt), traj0_response_ids=np.array(response), traj0_response_mask=np.array(mask),
             traj0_generation_spans=np.array(spans).reshape(-1, 2))
    return path


def test_recorded_rows_are_checked_and_never_truncated(tmp_path):
    good = _npz(tmp_path / "a.npz", [5, 6], [7, 8, 9, 10], [1, 1, 0, 1], [[0, 2], [3, 4]])
    row = ag.trajectory_row(good, max_length=10, vocab_size=20)
    assert row["loss_mask"] == [0, 0, 1, 1, 0, 1] and row["position_ids"] == list(range(6))
    with pytest.raises(OverflowError):
        ag.trajectory_row(good, max_length=5, vocab_size=20)
    with pytest.raises(ValueError, match="outside the student vocabulary"):
        ag.trajectory_row(good, max_length=10, vocab_size=10)
    with pytest.raises(ValueError, match="do not share"):
        ag.trajectory_row(good, max_length=10, vocab_size=20, excluded_token_ids=[8])
    with pytest.raises(ValueError, match="disagree"):
        ag.trajectory_row(_npz(tmp_path / "b.npz", [5], [7, 8], [1, 0], [[0, 2]]), max_length=10, vocab_size=20)
    with pytest.raises(ValueError, match="overlapping"):
        ag.trajectory_row(_npz(tmp_path / "c.npz", [5], [7, 8], [1, 1], [[1, 2], [0, 1]]), max_length=10, vocab_size=20)


def test_splits_tokenizers_and_packing(tmp_path):
    assert {ag.task_split("task-7", seed=s) for s in (1, 1, 1)} == {ag.task_split("task-7", seed=1)}
    share = sum(ag.task_split(f"t{i}") == "validation" for i in range(2000)) / 2000
    assert 0.07 < share < 0.13
    for name, extra in (("teacher", [{"id": 100, "content": "<tool>"}, {"id": 5, "content": "<eos>"}]), ("student", [{"id": 5, "content": "<eos>"}])):
        (tmp_path / name).mkdir()
        (tmp_path / name / "tokenizer.json").write_text(json.dumps({"model": {"vocab": {"a": 0}}, "added_tokens": extra}))
    report = ag.tokenizer_compatibility(tmp_path / "teacher", tmp_path / "student")
    assert report["excluded_token_ids"] == [100] and "tokenizer.json" in report["files"]["student"]
    (tmp_path / "student" / "tokenizer.json").write_text(json.dumps({"model": {"vocab": {"a": 1}}, "added_tokens": []}))
    with pytest.raises(ValueError, match="mismatch: model"):
        ag.tokenizer_compatibility(tmp_path / "teacher", tmp_path / "student")

    msgs = ag.normalize_tool_messages(episode(), system="s")
    row = ag.encode_assistant_targets(render, msgs, eos_token_id=EOS, max_length=200)
    (tmp_path / "rows.jsonl").write_text(json.dumps(row) + "\n" + json.dumps(row) + "\n")
    data = ag.PreparedTrajectories(tmp_path / "rows.jsonl", eos_token_id=EOS)
    assert len(data) == 2 and data.supervised_tokens() == 2 * sum(row["loss_mask"]) and data[0]["input_ids"].shape == data[0]["loss_mask"].shape
    from archlab_b200.train.sft import pack_examples

    x, y = pack_examples(data.examples(), row_len=len(row["input_ids"]) + 4)
    assert x.shape[0] == 2 and int((y >= 0).sum()) == data.supervised_tokens()
    with pytest.raises(ValueError, match="no supervised EOS"):
        ag.PreparedTrajectories([row], eos_token_id=77)
    with pytest.raises(ValueError, match="token / mask contract"):
        ag.PreparedTrajectories([{**row, "loss_mask": [1] + row["loss_mask"][1:]}])
