"""Frozen campaign tables: arm counts, sealed sizes, shared geometry and the size-dependent FineWeb templates."""
import pytest

from archlab_b200.contracts import campaigns as C


def test_ten_m_contract_and_geometry():
    assert C.verify_ten_m_contract() == {"variants": 16, "seeds": 3, "runs": 48}
    base = C.get_campaign_variant("10m", "baseline")
    assert base.parameter_count == 9_363_488 and base.steps == 286 and base.training_tokens == 286 * 192 * 2048
    kw = C.ten_m_model_config_kwargs(C.get_ten_m_variant("kda"))
    assert kw["depth"] == 5 and kw["aspect_ratio"] == 11 and kw["vocab_size"] == 32768 and kw["arch_family"] == "kimi_kda"
    assert kw["kda_pattern"] == "KKKG" and kw["per_head_muon"] is True
    assert C.get_campaign_variant("100m", "baseline").steps == 3228
    with pytest.raises(ValueError):
        C.get_campaign_variant("10m", "nope")
    with pytest.raises(ValueError):
        C.get_campaign_variant("1t", "baseline")


def test_fineweb_templates_scale_their_mechanisms():
    assert set(C.FINEWEB_CAMPAIGN_VARIANTS) == {"1m", "10m", "100m", "300m", "7b"}
    assert len(C.FINEWEB_CAMPAIGN_VARIANTS["100m"]) == 17                       # sixteen arms + colu
    eng = C.get_fineweb_variant_template("300m", "engram").model_kwargs()
    assert eng["engram_layers"] == (3, 9) and eng["engram_dim"] == 256 and eng["engram_num_heads"] == 8
    dsa = C.get_fineweb_variant_template("7b", "dsa").model_kwargs()
    assert (dsa["dsa_index_heads"], dsa["dsa_index_head_dim"], dsa["dsa_index_rope_dim"]) == (16, 128, 64)
    assert C.get_fineweb_variant_template("1m", "glm-mla").model_kwargs()["relative_dim"] == 4
    assert C.get_fineweb_variant_template("1m", "baseline").parameter_count == 0   # resolved from the built model
    kw = C.fineweb_model_config_kwargs("7b", C.get_fineweb_variant_template("7b", "colu"))
    assert kw["vocab_size"] == 50304 and kw["depth"] == 32 and kw["search_mlp"] == "colu"
    assert C.fineweb_token_budget("7b", 6_830_000_000) == 100_000_000_000
    assert C.fineweb_token_budget("10m", 10_000_000) == 120_000_000


@pytest.mark.parametrize("arm", ["baseline", "xielu", "kda", "attnres", "glm-mla", "partial-rope-25", "qwen-gdn", "engram", "mhc", "gated-attention", "dsa"])
def test_ten_m_arms_build_and_step(arm):
    import torch

    from archlab_b200.models.factory import build_campaign_arm, campaign_arm_config

    kw = C.ten_m_model_config_kwargs(C.get_ten_m_variant(arm))
    kw["vocab_size"], kw["max_seq_len"] = 512, 64                     # keep the test small; geometry stays 5 x 56, heads of 8
    family, cfg = campaign_arm_config(kw)
    assert cfg["n_layer"] == 5 and cfg["n_embd"] == 56 and cfg["n_head"] == 7
    model = build_campaign_arm(kw)
    ids = torch.randint(0, 512, (2, 64))
    loss = model(ids, ids)
    loss = loss[0] if isinstance(loss, tuple) else loss
    loss.backward()
    assert torch.isfinite(loss)


def test_unknown_family_is_refused_by_name():
    from archlab_b200.models.factory import campaign_arm_config

    with pytest.raises(NotImplementedError):
        campaign_arm_config({"arch_family": "made_up", "depth": 2, "aspect_ratio": 8, "head_dim": 8})


def test_dsa_stages():
    import torch

    from archlab_b200.models.factory import build_campaign_arm

    kw = C.ten_m_model_config_kwargs(C.get_ten_m_variant("dsa"))
    kw["vocab_size"], kw["max_seq_len"] = 512, 64
    model = build_campaign_arm(kw)
    ids = torch.randint(0, 512, (2, 64))
    dense = model(ids, ids)
    model.set_stage("sparse")
    sparse = model(ids, ids)
    sparse.backward()
    assert torch.isfinite(dense) and torch.isfinite(sparse) and dense.item() != sparse.item()
    assert all(p.grad is not None for p in model.indexer_parameters())
    model.eval()
    assert model(ids).shape == (2, 64, 512)


def test_every_frozen_run_command_parses_and_names_a_buildable_arm():
    from archlab_b200.contracts.registry import campaign_grid
    from archlab_b200.models.factory import campaign_arm_config
    from archlab_b200.train import base_train

    seen = set()
    for run in campaign_grid():
        if run.variant_id in seen:
            continue
        seen.add(run.variant_id)
        argv = run.command()[3:]                                   # after "python -m archlab_b200.train.base_train"
        a = base_train.parse_args(argv)
        assert a.depth == run.depth and a.num_iterations == run.steps
        family, cfg = campaign_arm_config(base_train.arm_model_kwargs(a))
        assert cfg["n_layer"] == run.depth
    assert len(seen) == 16


def test_arm_path_trains_through_the_mesh_trainer(tmp_path, monkeypatch):
    import json

    from archlab_b200.train import base_train

    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    rc = base_train.main(["--arch-family=kimi_kda", "--depth=2", "--aspect-ratio=16", "--head-dim=8", "--max-seq-len=32",
                          "--vocab-size=256", "--device-batch-size=2", "--total-batch-size=128", "--num-iterations=3",
                          "--kda-pattern=KG", "--kda-force-final-global", "--model-tag=arm", f"--run-dir={tmp_path}"])
    assert rc == 0
    rows = [json.loads(l) for l in open(tmp_path / "arm" / "metrics_rank0.jsonl")]
    assert len(rows) == 3 and all(r["loss"] == r["loss"] for r in rows)
