"""Reasoning-chat rendering around a pinned encoder: fragment repair, prefix-stable spans, token boundaries."""
import hashlib

import pytest

from archlab_b200.data import chat_render as cr


def encode(messages):
    out = "<bos>"
    for m in messages:
        if m["role"] == "assistant":
            out += "<a><think>" + (m.get("reasoning_content") or "") + "</think>" + m.get("content", "") + ("<call>" if m.get("tool_calls") else "") + "<eos>"
        else:
            out += f"<{m['role'][0]}>" + m.get("content", "")
    return out


def test_reasoning_only_fragments_are_joined_and_everything_else_is_kept():
    msgs = [{"role": "user", "content": "q"}, {"role": "assistant", "reasoning_content": "first"},
            {"role": "assistant", "reasoning_content": "second", "content": "answer"}]
    merged, repairs = cr.coalesce_reasoning_fragments(msgs)
    assert len(merged) == 2 and merged[1]["reasoning_content"] == "first\n\nsecond" and merged[1]["content"] == "answer"
    assert repairs[0]["policy"] == "merge-reasoning-only-prefixes" and repairs[0]["source_message_indices"] == [1, 2]
    assert repairs[0]["reasoning_sha256"][0] == hashlib.sha256(b"first").hexdigest()
    two_answers = [{"role": "user", "content": "q"}, {"role": "assistant", "content": "a1"}, {"role": "assistant", "content": "a2"}]
    kept, repairs = cr.coalesce_reasoning_fragments(two_answers)
    assert kept == two_answers and repairs[0]["messages_merged"] is False
    with pytest.raises(ValueError, match="cannot discard"):
        cr.coalesce_reasoning_fragments([{"role": "user", "content": "q"}, {"role": "assistant", "reasoning_content": "r", "name": "x"},
                                         {"role": "assistant", "content": "a"}])
    same, none = cr.coalesce_reasoning_fragments(two_answers[:2])
    assert same == two_answers[:2] and none == []


def test_spans_cover_exactly_what_each_assistant_turn_adds():
    msgs = [{"role": "user", "content": "q1"}, {"role": "assistant", "reasoning_content": "r", "content": "a1"},
            {"role": "user", "content": "q2"}, {"role": "assistant", "content": "a2"}]
    text, merged, meta = cr.render_conversation(encode, msgs, bos="<bos>", eos="<eos>")
    spans = meta["assistant_character_spans"]
    assert [text[a:b] for a, b in spans] == ["<a><think>r</think>a1<eos>", "<a><think></think>a2<eos>"] and "message_repairs" not in meta
    _, _, flagged = cr.render_conversation(encode, msgs[:3], bos="<bos>")
    assert flagged["message_repairs"][0]["policy"] == "keep-non-assistant-ending"
    with_call = msgs[:1] + [{"role": "assistant", "content": "", "tool_calls": [{"id": "c"}]}]
    assert cr.render_conversation(encode, with_call)[2]["message_repairs"][0]["policy"] == "keep-terminal-tool-call"
    _, with_tools, _ = cr.render_conversation(encode, msgs, tools=[{"name": "bash"}])
    assert with_tools[0] == {"role": "system", "content": "", "tools": [{"name": "bash"}]}

    def unstable(messages):
        return encode(messages) if len(messages) < 4 else encode(messages).replace("q1", "Q1")
    with pytest.raises(ValueError, match="prefix-stable"):
        cr.render_conversation(unstable, msgs)
    with pytest.raises(ValueError, match="explicit policy"):
        cr.render_conversation(encode, [{"role": "assistant", "content": "a"}])
    with pytest.raises(ValueError, match="text-only"):
        cr.render_conversation(encode, [{"role": "user", "content": [{"type": "image"}]}])


def test_token_spans_fail_closed_on_merges_across_a_boundary():
    offsets = [(0, 5), (5, 8), (8, 10), (10, 14), (14, 20)]
    assert cr.token_spans(offsets, [(5, 10), (14, 20)]) == [[1, 3], [4, 5]]
    with pytest.raises(ValueError, match="crosses"):
        cr.token_spans(offsets, [(6, 10)])
    with pytest.raises(ValueError, match="crosses"):
        cr.token_spans(offsets, [(5, 9)])
    with pytest.raises(ValueError, match="overlaps"):
        cr.token_spans([(0, 6), (5, 8)], [(5, 8)])


def test_encoder_files_are_pinned_by_hash(tmp_path):
    f = tmp_path / "encoding.py"
    f.write_text("bos_token = '<bos>'\ndef encode_messages(m):\n    return bos_token + str(len(m))\n")
    digest = hashlib.sha256(f.read_bytes()).hexdigest()
    module = cr.load_pinned_encoder(f, digest)
    assert module.encode_messages([1, 2]) == "<bos>2"
    with pytest.raises(ValueError, match="reviewed revision"):
        cr.load_pinned_encoder(f, "0" * 64)
