"""CPU plumbing: scheduler + prefix cache + reference engine on the fp32 2-layer decoder, single rank and
tensor-parallel over gloo (two processes on 127.0.0.1)."""
import json
import subprocess
import sys

import torch


def _run(world, requests=12, max_tokens=6):
    out = subprocess.run([sys.executable, "-m", "dgpp_b200.engine.plumbing", "--requests", str(requests),
                          "--max-tokens", str(max_tokens), "--world", str(world)],
                         capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    return [json.loads(l) for l in out.stdout.strip().splitlines() if l.startswith("{")]


def test_single_rank_is_deterministic_and_hits_prefix_cache():
    a, b = _run(1)[0], _run(1)[0]
    assert a["tokens_sha256"] == b["tokens_sha256"] and a["op_digest"] == b["op_digest"]
    assert a["prefix_hit_tokens"] > 0


def test_tp2_over_gloo_matches_on_every_rank():
    ranks = _run(2)
    assert len(ranks) == 2
    assert ranks[0]["tokens_sha256"] == ranks[1]["tokens_sha256"]
    assert ranks[0]["op_digest"] == ranks[1]["op_digest"]
    assert ranks[0]["prefix_digest"] == ranks[1]["prefix_digest"]


def test_prefix_hit_equals_cold_prefill():
    from dgpp_b200.engine.adapters import ReferenceEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel
    from dgpp_b200.ops import reference as ref
    from dgpp_b200.runtime import rt

    cfg = DenseConfig.plumbing_fp32()
    m = DenseModel.random_init(cfg, device="cpu", seed=0, std=0.02)
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 4096, (64,), generator=g).tolist()
    prompts = {f"r{i}": shared + torch.randint(0, 4096, (10 + i,), generator=g).tolist() for i in range(3)}

    def tokens(prefix_cache):
        with ref.activation_dtype(torch.float32):
            eng = ReferenceEngine(m, slots=1, num_blocks=64, block_tokens=16, max_context=256)
            sc = rt.SchedulerConfig()
            sc.prefix_cache = prefix_cache
            s = rt.Scheduler(eng, sc)
            for rid, p in prompts.items():
                s.submit(rid, p, 5)
            s.run(10000)
            out = {}
            for kind, rid, a, b in s.events():
                if kind == "token":
                    out.setdefault(rid, []).append(a)
            return out, s.meters()["prefix_hit_tokens"]

    hot, hits = tokens(True)
    cold, none = tokens(False)
    assert hits >= 2 * 64 and none == 0
    assert hot == cold
