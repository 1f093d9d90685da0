"""Audit of a git revision before it is published: only the committed tree is read, never the work tree.

    python -m archlab_b200.services.publication_audit --root . --revision HEAD --output audit.json

Every blob of the revision is checked against a small table of rules (what the reference's audit enforces,
src/archlab/reporting/publication_audit.py:38-128): it must live under an approved root, must not sit inside a workspace
or credential directory, must not be a data / weight / log / key file, must be a regular file (no symlinks, no
unregistered submodules), must stay under a size limit and must not contain credential patterns.  Findings name the
path and the rule, never the matched bytes.  The result carries a (path, size, sha256) manifest of the audited tree, so
the published archive can be compared with what was audited; the exit code is 1 when anything was found.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import re
import subprocess
from dataclasses import dataclass, field
from pathlib import Path, PurePosixPath
from typing import Callable

REGULAR_MODES = frozenset({"100644", "100755"})
GITLINK_MODE = "160000"


@dataclass(frozen=True)
class Policy:
    roots: frozenset = frozenset({".github", "archlab_b200", "baseline", "tests", "recipes", "profiles", "docs"})
    # top-level files: documents, project metadata and the two entry scripts, by suffix; dot-files by name
    root_suffixes: tuple = (".md", ".json", ".toml", ".py", ".cff")
    root_files: frozenset = frozenset({".gitmodules", ".python-version", "LICENSE"})       # plus any top-level ".*ignore*" file
    workspace_parts: frozenset = frozenset({".git", ".aws", ".ssh", ".venv", "__pycache__", "node_modules", "results", "runs",
                                            "checkpoints", "mlruns", "wandb", "_ref"})
    payload_suffixes: tuple = (".pt", ".pth", ".ckpt", ".safetensors", ".bin", ".idx", ".parquet", ".arrow", ".jsonl", ".jsonl.gz",
                               ".log", ".pem", ".key", ".p12", ".pickle", ".pkl", ".so", ".o", ".ncu-rep")
    max_blob_bytes: int = 5 * 1024 * 1024
    submodules: dict = field(default_factory=dict)         # path -> (name, url) of registered submodules
    secrets: dict = field(default_factory=lambda: {
        "private_key": re.compile(rb"-----BEGIN (?:RSA |EC |OPENSSH )?PRIVATE KEY-----"),
        "github_token": re.compile(rb"\b(?:gh[pousr]_[A-Za-z0-9]{36,}|github_pat_[A-Za-z0-9_]{40,})\b"),
        "aws_access_key": re.compile(rb"\b(?:AKIA|ASIA)[A-Z0-9]{16}\b"),
        "credential_url": re.compile(rb"https?://[^\s/:@]+:[^\s/@]+@"),
    })


@dataclass(frozen=True)
class Blob:
    path: str
    mode: str
    content: bytes

    @property
    def parts(self) -> tuple:
        return PurePosixPath(self.path).parts


# rule name -> predicate(blob, policy) that is true when the blob violates it
RULES: dict[str, Callable[[Blob, Policy], bool]] = {
    "unapproved_root": lambda b, p: not b.parts or not (
        b.parts[0] in p.roots or (len(b.parts) == 1 and (b.path in p.root_files or (b.path.startswith(".") and "ignore" in b.path)
                                                         or (b.path.endswith(p.root_suffixes) and not b.path.startswith("."))))),
    "workspace_artifact": lambda b, p: any(part in p.workspace_parts for part in b.parts),
    "data_or_secret_file": lambda b, p: b.path.endswith(p.payload_suffixes)
    or (b.parts[-1].startswith(".env") and b.parts[-1] != ".env.example"),
    "non_regular_file": lambda b, p: b.mode not in REGULAR_MODES,
    "oversize_blob": lambda b, p: len(b.content) > p.max_blob_bytes,
}


def inspect_blob(blob: Blob, policy: Policy = Policy()) -> list[str]:
    """Names of the violated rules (path rules first, then credential patterns); matched bytes are never returned."""
    reasons = [name for name, violated in RULES.items() if violated(blob, policy)]
    return reasons + [name for name, pattern in policy.secrets.items() if pattern.search(blob.content)]


class _Tree:
    def __init__(self, root: Path, revision: str):
        self.root = Path(root)
        self.commit = self.git("rev-parse", "--verify", f"{revision}^{{commit}}").decode().strip()

    def git(self, *args: str, stdin: bytes | None = None) -> bytes:
        return subprocess.run(["git", "-C", str(self.root), *args], input=stdin, capture_output=True, check=True).stdout

    def entries(self):
        """(mode, kind, object id, path) of every entry of the revision, recursively."""
        for record in filter(None, self.git("ls-tree", "-rz", self.commit).split(b"\0")):
            head, path = record.split(b"\t", 1)
            mode, kind, oid = head.decode().split()
            yield mode, kind, oid, path.decode()

    def contents(self, oids: list[str]):
        """Blob bytes in the order asked, from one ``cat-file --batch`` process."""
        stream = self.git("cat-file", "--batch", stdin="".join(f"{oid}\n" for oid in oids).encode())
        at = 0
        for oid in oids:
            eol = stream.index(b"\n", at)
            got, kind, size = stream[at:eol].decode().split()
            if (got, kind) != (oid, "blob"):
                raise ValueError("unexpected object in the publication tree")
            yield stream[eol + 1:eol + 1 + int(size)]
            at = eol + 1 + int(size) + 1


def audit_tree(root, revision: str = "HEAD", policy: Policy = Policy()) -> dict:
    tree = _Tree(root, revision)
    blobs, findings, submodules = [], [], []
    for mode, kind, oid, path in tree.entries():
        if kind == "blob":
            blobs.append((mode, oid, path))
        elif kind == "commit" and mode == GITLINK_MODE:
            if path in policy.submodules:
                name, url = policy.submodules[path]
                submodules.append({"name": name, "path": path, "url": url, "revision": oid})
            else:
                findings.append({"path": path, "reasons": ["unapproved_submodule"]})
        else:
            raise ValueError("publication tree contains an unsupported object")
    manifest = []
    for (mode, oid, path), content in zip(blobs, tree.contents([oid for _, oid, _ in blobs])):
        manifest.append({"path": path, "bytes": len(content), "sha256": hashlib.sha256(content).hexdigest()})
        if reasons := inspect_blob(Blob(path, mode, content), policy):
            findings.append({"path": path, "reasons": reasons})
    return {"revision": tree.commit, "passed": not findings, "files": len(manifest), "bytes": sum(m["bytes"] for m in manifest),
            "findings": findings, "manifest": manifest, "submodules": submodules,
            "scope": "the selected git tree and registered submodule pins only; ignored local files are not read"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--root", type=Path, default=Path.cwd())
    ap.add_argument("--revision", default="HEAD")
    ap.add_argument("--output", type=Path, required=True)
    a = ap.parse_args(argv)
    result = audit_tree(a.root, a.revision)
    a.output.write_text(json.dumps(result, indent=2) + "\n")
    print(json.dumps({k: result[k] for k in ("revision", "passed", "files", "bytes", "findings")}))
    return 0 if result["passed"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
