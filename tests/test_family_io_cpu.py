"""Native family checkpoints: write a random-init model of every family, load it back, same oracle logits; refusals
name the tensor."""
import json
import os

import pytest
import torch

from dgpp_b200.loaders.family_io import load_family, save_family
from dgpp_b200.models.moe import MoEConfig


def _models():
    from dgpp_b200.models.dory import DoryConfig, DoryModel
    from dgpp_b200.models.engram import EngramConfig
    from dgpp_b200.models.flash_next import FlashNextConfig, FlashNextModel, QsaConfig
    from dgpp_b200.models.glm_flash import GlmFlashConfig, GlmFlashModel
    from dgpp_b200.models.mimo import MimoConfig, MimoModel
    from dgpp_b200.models.minimax import MinimaxConfig, MinimaxModel

    moe = MoEConfig(hidden=256, experts=4, top_k=2, moe_ffn=256, shared_ffn=256)
    yield "glm_flash", GlmFlashModel.random_init(
        GlmFlashConfig(layers=2, hidden=256, vocab=512, mla_every=2, k_heads=2, v_heads=2, dk=64, dv=64, heads=4, q_lora=128,
                       kv_lora=64, nope=32, rope=32, v_dim=32, ffn=512, moe=moe, engram=EngramConfig(bucket=200),
                       engram_layers=(1,)), "cpu", seed=3)
    yield "dory", DoryModel.random_init(DoryConfig(hidden=256, head_dim=64, ffn=512, vocab=512, loops=2), "cpu", seed=3)
    yield "flash_next", FlashNextModel.random_init(
        FlashNextConfig(layers=2, hidden=256, full_every=2, q_heads=4, kv_heads=2, head_dim=64, gdn_k_heads=2, gdn_v_heads=2,
                        gdn_dk=64, gdn_dv=64, ffn=512, vocab=512, gr_rank=64, ple_rows=128, page=8,
                        qsa=QsaConfig(index_heads=2, index_dim=64, select_k=1)), "cpu", seed=3)
    mm = MoEConfig(hidden=256, experts=4, top_k=2, moe_ffn=256, shared_ffn=256, swiglu_limit=7.0, swiglu_alpha=1.702)
    yield "minimax", MinimaxModel.random_init(
        MinimaxConfig(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, rotary_dim=32, index_dim=64, sparse_block=8,
                      sparse_topk=2, dense_ffn=512, vocab=512, moe=mm, moe_layers=[False, True]), "cpu", seed=3)
    yield "mimo", MimoModel.random_init(
        MimoConfig(layers=2, hidden=256, q_heads=4, kv_heads=1, swa_kv_heads=2, head_dim=64, rotary_dim=32, window=8,
                   ffn=512, vocab=512, swa_layers=[True, False],
                   moe=MoEConfig(hidden=256, experts=4, top_k=2, moe_ffn=256)), "cpu", seed=3)


@pytest.mark.parametrize("family", ["glm_flash", "dory", "flash_next", "minimax", "mimo"])
def test_round_trip_keeps_the_oracle_logits(tmp_path, family):
    model = dict(_models())[family]
    out = str(tmp_path / family)
    save_family(model, out)
    cfg = json.load(open(os.path.join(out, "config.json")))
    assert cfg["model_type"] == f"dgpp-{family}" and cfg["quant"]
    back = load_family(out, "cpu")
    assert type(back) is type(model) and back.cfg == model.cfg
    t = torch.randint(0, 512, (20,), generator=torch.Generator().manual_seed(1))
    assert torch.equal(back.forward_reference(t), model.forward_reference(t))
    if family == "mimo":
        _, h = model.forward_reference(t, return_hidden=True)
        assert torch.equal(back.draft_reference(h[:19], t[1:]), model.draft_reference(h[:19], t[1:]))


def test_refusals_name_the_tensor(tmp_path):
    from dgpp_b200.loaders.checkpoint import open_checkpoint, write_safetensors

    model = dict(_models())["dory"]
    out = str(tmp_path / "d")
    save_family(model, out)
    ck = open_checkpoint(out)
    tensors = {n: ck.tensor(n).clone() for n in ck.names()}
    victim = next(n for n in tensors if n.endswith("payload"))
    bad = str(tmp_path / "bad")
    os.makedirs(bad)
    open(os.path.join(bad, "config.json"), "w").write(open(os.path.join(out, "config.json")).read())
    write_safetensors(os.path.join(bad, "model.safetensors"), {n: t for n, t in tensors.items() if n != victim})
    with pytest.raises(ValueError, match=victim.rsplit(".", 1)[0].replace(".", r"\.")):
        load_family(bad, "cpu")
    tensors["stray.tensor"] = torch.zeros(3)
    write_safetensors(os.path.join(bad, "model.safetensors"), tensors)
    with pytest.raises(ValueError, match="stray"):
        load_family(bad, "cpu")
    cfg = json.load(open(os.path.join(out, "config.json")))
    cfg["model_type"] = "llama"
    open(os.path.join(bad, "config.json"), "w").write(json.dumps(cfg))
    with pytest.raises(ValueError, match="native family"):
        load_family(bad, "cpu")


def test_fixture_writer_cli(tmp_path, capsys):
    from dgpp_b200.loaders.family_io import main

    assert main(["--family", "dory", "--out", str(tmp_path / "fx"), "--vocab", "512", "--check"]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["family"] == "dory" and rep["round_trip_equal"] is True and rep["tensors"] > 10
    assert os.path.exists(tmp_path / "fx" / "model.safetensors")
