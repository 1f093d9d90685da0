"""Preregistered repeated-data sweep: the grid, its order, canonical names, the derived plan."""
import json

import pytest

from archlab_b200.train import loop_sweep as ls


def test_grid_is_fixed_and_ordered():
    cells = ls.cells()
    assert len(cells) == sum(len(v) for v in ls.GRID.values()) * len(ls.WEIGHT_DECAYS) == 37 * 6
    first = cells[0]
    assert (first["reference_depth"], first["recursions"], first["weight_decay"]) == ls.ANCHOR and first["stored_layers"] == 20 and first["hidden_size"] == 128
    main = [c for c in cells if c["weight_decay"] == 0.8]
    assert cells[:len(main)] == main and all(c["weight_decay"] != 0.8 for c in cells[len(main):])
    assert {c["hidden_size"] for c in cells} == {128, 256, 384} and ls.make_cell(18, 1, 0.8)["stored_layers"] == 45
    assert ls.cell_name(first) == "loop-d128-L20-K2-wd0p8" and len({ls.cell_name(c) for c in cells}) == len(cells)
    assert len(ls.cells_sha256()) == 64 and ls.cells_sha256() == ls.cells_sha256()
    for bad in ({**first, "recursions": 5}, {**first, "weight_decay": 0.3}, {**first, "epochs": 3}, {**first, "hidden_size": 256}):
        with pytest.raises(ValueError, match="preregistered"):
            ls.validate_cell(bad)


def test_plan_has_one_isolated_run_per_cell(tmp_path):
    base = {"root": str(tmp_path / "campaign"), "environment": {"PYTHONPATH": "/old/src:/third_party", "NCCL_DEBUG": "WARN"},
            "runs": [{"variant": "simplicial", "width": 128}, {"variant": "normal", "width": 128, "extra_args": ["--depth", "20"], "nodes": 1}]}
    (tmp_path / "base.json").write_text(json.dumps(base))
    plan = ls.write_plan(tmp_path / "base.json", source=tmp_path / "checkout", commit="abc123", destination=tmp_path / "plan.json")
    runs = plan["runs"]
    assert len(runs) == 222 and plan["planned_training_tokens"] == 222 * 10 ** 9 and plan["cells_sha256"] == ls.cells_sha256()
    assert len({r["master_port"] for r in runs}) == len({r["output"] for r in runs}) == 222
    r = runs[0]
    assert r["nodes"] == 1 and r["extra_args"][:2] == ["--depth", "20"] and r["extra_args"][2] == "--sweep-cell"
    assert json.loads(open(r["extra_args"][3]).read()) == r["cell"] and r["environment"]["PYTHONPATH"] == f"{tmp_path / 'checkout'}:/third_party"
    assert base["environment"]["PYTHONPATH"] == "/old/src:/third_party" and json.loads((tmp_path / "plan.json").read_text())["format"] == plan["format"]
