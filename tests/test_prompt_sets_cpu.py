"""Versioned prompt sets."""
import pytest

from archlab_b200.contracts import prompts as P


def test_default_set_and_tag_filter():
    ps = P.load_prompt_set()
    assert len(ps) == 7 and len({p.id for p in ps}) == 7 and all(p.text for p in ps)
    assert P.prompt_texts(tag="math") == ["If 3*x - 4 = 11, then x is"]


@pytest.mark.parametrize("body,message", [
    ("schema_version: 2\nprompts: [{id: a, text: b}]\n", "unsupported prompt schema"),
    ("schema_version: 1\nprompts: []\n", "empty"),
    ("schema_version: 1\nprompts: [{id: a, text: b}, {id: a, text: c}]\n", "invalid or duplicate prompt 'a'"),
    ("schema_version: 1\nprompts: [{id: a, text: ''}]\n", "invalid or duplicate"),
    ("schema_version: 1\nprompts: [{id: a, text: b, tags: [1]}]\n", "invalid tags"),
    ("schema_version: 1\nprompts: [just text]\n", "invalid prompt row"),
])
def test_malformed_sets_are_refused_by_name(tmp_path, body, message):
    f = tmp_path / "set.yaml"
    f.write_text(body)
    with pytest.raises(ValueError, match=message) as err:
        P.load_prompt_set(f)
    assert str(f) in str(err.value)


def test_training_loop_reads_versioned_sets(tmp_path):
    from archlab_b200.train.evaluation import load_prompts

    class Tok:
        def encode(self, text, prepend_bos=False):
            return [1] * prepend_bos + [ord(c) % 50 + 2 for c in text]

    out = load_prompts(P.DEFAULT_SET, Tok())
    assert len(out) == 7 and all(p[0] == 1 for p in out)
