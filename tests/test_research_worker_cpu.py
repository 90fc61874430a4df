"""Research socket worker on CPU: every operation against the model's oracle called directly."""
import base64
import threading

import numpy as np
import pytest
import torch

from dgpp_b200.adapters.lora import random_adapter_tensors, save_adapter
from dgpp_b200.models.dense import DenseConfig, DenseModel
from dgpp_b200.tools.research_worker import ResearchServer, ResearchWorld, request


@pytest.fixture(scope="module")
def served():
    cfg = DenseConfig.tiny(vocab=512, weight_fmt="bf16")
    model = DenseModel.random_init(cfg, device="cpu", seed=2, std=0.05)
    srv = ResearchServer(ResearchWorld(model), port=0, token="s3")
    th = threading.Thread(target=srv.serve_forever, daemon=True)
    th.start()
    yield model, srv.port
    assert request(srv.port, {"op": "shutdown", "token": "s3"})["ok"]
    th.join(timeout=10)


def _arr(d):
    return np.frombuffer(base64.b64decode(d["b64"]), np.float32).reshape(d["shape"])


def test_logits_generate_likelihood_capture(served):
    model, port = served
    toks = torch.randint(0, 512, (12,), generator=torch.Generator().manual_seed(0)).tolist()
    want, _ = model.forward_reference(torch.tensor(toks))
    r = request(port, {"op": "logits", "tokens": toks, "top_k": 3, "full": True, "token": "s3"})
    assert r["ok"] and np.array_equal(_arr(r["logits"]), want[-1].float().numpy())
    assert [t["id"] for t in r["top"]] == torch.argsort(-want[-1].float(), stable=True)[:3].tolist()
    assert abs(r["top"][0]["logprob"] - float(torch.log_softmax(want[-1].float(), -1).max())) < 1e-5
    # greedy generation = repeated argmax over the growing prompt
    g = request(port, {"op": "generate", "tokens": toks, "max_new": 4, "token": "s3"})["tokens"]
    cur = list(toks)
    for t in g:
        lg, _ = model.forward_reference(torch.tensor(cur))
        assert t == int(torch.argsort(-lg[-1].float(), stable=True)[0])
        cur.append(t)
    assert request(port, {"op": "generate", "tokens": toks, "max_new": 4, "stop": [g[1]], "token": "s3"})["tokens"] == g[:2]
    # teacher-forced likelihood
    lk = request(port, {"op": "likelihood", "tokens": toks, "start": 5, "token": "s3"})
    lp = torch.log_softmax(want[:-1].float(), -1)
    per = [float(lp[i - 1, toks[i]]) for i in range(5, 12)]
    assert lk["count"] == 7 and np.allclose(lk["per_token"], per, atol=1e-5) and abs(lk["logprob"] - sum(per)) < 1e-4
    # activations: the stream entering a layer and the final-norm input
    L = model.cfg.layers
    cap = {1: None, L: None}
    model.forward_reference(torch.tensor(toks), capture=cap)
    c = request(port, {"op": "capture", "tokens": toks, "layers": [1, L], "rows": "all", "token": "s3"})["activations"]
    assert np.array_equal(_arr(c["1"]), cap[1].float().numpy()) and np.array_equal(_arr(c[str(L)]), cap[L].float().numpy())
    last = request(port, {"op": "capture", "tokens": toks, "layers": [1], "token": "s3"})["activations"]["1"]
    assert last["shape"] == [1, model.cfg.hidden]
    info = request(port, {"op": "info", "token": "s3"})
    assert info["layers"] == L and info["vocab"] == 512 and info["adapter"] is False


def test_adapter_install_and_errors(served, tmp_path):
    model, port = served
    toks = list(range(3, 13))
    base = request(port, {"op": "logits", "tokens": toks, "full": True, "token": "s3"})
    tensors = random_adapter_tensors(model.cfg, 4, ["q_proj", "v_proj", "down_proj"], seed=1, std=0.2)
    save_adapter(str(tmp_path / "ad"), tensors, 4, 8.0, ["q_proj", "v_proj", "down_proj"])
    ins = request(port, {"op": "install_adapter", "dir": str(tmp_path / "ad"), "token": "s3"})
    assert ins["ok"] and ins["rank"] == 4
    with_ad = request(port, {"op": "logits", "tokens": toks, "full": True, "token": "s3"})
    assert np.abs(_arr(with_ad["logits"]) - _arr(base["logits"])).max() > 1e-3
    assert request(port, {"op": "info", "token": "s3"})["adapter"] is True
    assert request(port, {"op": "remove_adapter", "token": "s3"})["ok"]
    again = request(port, {"op": "logits", "tokens": toks, "full": True, "token": "s3"})
    assert np.array_equal(_arr(again["logits"]), _arr(base["logits"]))
    # failures answer and leave the worker serving
    assert "bad token" in request(port, {"op": "info"})["error"]
    assert "unknown op" in request(port, {"op": "nope", "token": "s3"})["error"]
    assert "tokens" in request(port, {"op": "logits", "tokens": [1, 99999], "token": "s3"})["error"]
    assert "layers" in request(port, {"op": "capture", "tokens": toks, "layers": [77], "token": "s3"})["error"]
    assert "start" in request(port, {"op": "likelihood", "tokens": toks, "start": 0, "token": "s3"})["error"]
    assert request(port, {"op": "info", "token": "s3"})["ok"]
    with pytest.raises(ValueError):
        ResearchServer(ResearchWorld(model), host="0.0.0.0")


def test_family_models_answer_logits_generation_and_likelihood():
    from dgpp_b200.models.mimo import MimoConfig, MimoModel
    from dgpp_b200.tools.research_worker import FamilyWorld

    m = MimoModel.random_init(MimoConfig(layers=2, hidden=256, q_heads=4, kv_heads=1, swa_kv_heads=2, head_dim=64, rotary_dim=32,
                                         window=8, ffn=512, vocab=512, swa_layers=[True, False]), "cpu", seed=1)
    w = FamilyWorld(m)
    toks = torch.randint(0, 512, (10,), generator=torch.Generator().manual_seed(3)).tolist()
    want = m.forward_reference(torch.tensor(toks))
    r = w.handle({"op": "logits", "tokens": toks, "top_k": 2})
    assert r["top"][0]["id"] == int(torch.argsort(-want[-1].float(), stable=True)[0])
    g = w.handle({"op": "generate", "tokens": toks, "max_new": 3})["tokens"]
    cur = list(toks)
    for t in g:
        assert t == int(torch.argsort(-m.forward_reference(torch.tensor(cur))[-1].float(), stable=True)[0])
        cur.append(t)
    lk = w.handle({"op": "likelihood", "tokens": toks, "start": 4})
    lp = torch.log_softmax(want[:-1].float(), -1)
    assert abs(lk["logprob"] - sum(float(lp[i - 1, toks[i]]) for i in range(4, 10))) < 1e-4
    assert w.handle({"op": "info"})["family"] == "MimoModel"
    with pytest.raises(ValueError, match="unknown op"):
        w.handle({"op": "capture", "tokens": toks, "layers": [0]})
