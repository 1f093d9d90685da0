"""Sandbox gate: an agent tool call runs isolated, and a task verifier accepts a correct solution only."""
from archlab_b200.train.local_sandbox import LocalSandbox


def test_agent_tool_and_successful_verifier():
    with LocalSandbox(wall_seconds=10) as sb:
        r = sb.run_python("import os\nopen('answer.txt', 'w').write(str(sum(range(101))))\nprint(sorted(os.environ))")
        assert r.returncode == 0 and "HOME" not in r.stdout and "PATH" in r.stdout
        checker = "import sys\nsys.exit(0 if open('answer.txt').read().strip() == '5050' else 1)"
        assert sb.verify(checker)
        sb.write("answer.txt", "41")
        assert not sb.verify(checker)
        slow = sb.run_python("while True: pass")
        assert slow.timed_out or slow.returncode != 0
        try:
            sb.write("../escape.txt", "x")
            raise AssertionError("path escape must be refused")
        except ValueError:
            pass
