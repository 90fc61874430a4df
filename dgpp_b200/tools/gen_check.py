"""Offline generation check: run prompts through the kernel engine and through the PyTorch oracle of the same
weights, report where greedy tokens agree and how far the logits are apart, and (optionally) time the run.

    python -m dgpp_b200.tools.gen_check --model <checkpoint dir | org/name | tiny | 27b> [--layers N]
           [--prompt-lens 70,333] [--tokens 16] [--teacher-forced] [--json]

For every prompt the engine generates `--tokens` tokens; the oracle is then run teacher-forced over prompt +
generated tokens.  Reported per prompt: the first step at which the engine's token is not the oracle's argmax (-1 =
never), the oracle's margin at that step (a near tie is a legitimate difference between two correct
implementations), the oracle log-likelihood of the generated continuation, and the maximum logit difference of the
first generated position.  Exit status 1 when a divergence happens at a margin above `--tie`.
(reference counterparts: apps/glm_gen_check.cpp offline generation / benchmark harness, the per-family
 *_forward_check / *_load_check apps, and the teacher-forced likelihood of apps/dgpp_heretic_worker.cpp.)
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def build_model(spec: str, layers: int, device: str):
    from ..models.dense import DenseConfig, DenseModel
    if spec == "tiny":
        cfg = DenseConfig.tiny(hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=4096, layers=layers or 2)
        return DenseModel.random_init(cfg, device=device, seed=0, std=0.05)
    if spec == "27b":
        return DenseModel.random_init(DenseConfig.dense_27b(layers=layers or 2), device=device, seed=0)
    from ..loaders.checkpoint import load_dense
    return load_dense(spec, device=device)


def check(model, prompt_lens, n_tokens: int, tie: float, device: str):
    from ..engine.llm_engine import LLMEngine
    cfg = model.cfg
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in prompt_lens]
    eng = LLMEngine(model, max_batch=len(prompts), max_seq_len=max(prompt_lens) + n_tokens + 64,
                    prefill_chunk=min(2048, max(64, max(prompt_lens))))
    t0 = time.time()
    outs = eng.generate(prompts, max_tokens=n_tokens)
    torch.cuda.synchronize()
    wall = time.time() - t0
    rows = []
    for p, got in zip(prompts, outs):
        toks = torch.tensor(p + got[:-1], device=device)
        logits, _ = model.forward_reference(toks)
        lg = logits[len(p) - 1:].float()                          # position i predicts generated token i
        logp = torch.log_softmax(lg, -1)
        ll = float(sum(logp[i, t] for i, t in enumerate(got)))
        first_bad, margin = -1, 0.0
        for i, t in enumerate(got):
            top2 = torch.topk(lg[i], 2)
            if int(top2.indices[0]) != t:
                first_bad = i
                margin = float(top2.values[0] - lg[i, t])
                break
        rows.append({"prompt_len": len(p), "tokens": len(got), "first_divergence": first_bad,
                     "oracle_margin_there": round(margin, 5), "oracle_loglik": round(ll, 4),
                     "ok": first_bad < 0 or margin <= tie})
    return {"model": cfg.name, "layers": cfg.layers, "wall_s": round(wall, 3), "prompts": rows,
            "ok": all(r["ok"] for r in rows)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--prompt-lens", default="70,333")
    ap.add_argument("--tokens", type=int, default=16)
    ap.add_argument("--tie", type=float, default=0.05, help="largest oracle margin still counted as a near tie")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("gen_check drives the kernel engine and needs a GPU", file=sys.stderr)
        return 2
    model = build_model(a.model, a.layers, "cuda")
    rep = check(model, [int(x) for x in a.prompt_lens.split(",")], a.tokens, a.tie, "cuda")
    if a.json:
        print(json.dumps(rep))
    else:
        print(f"{rep['model']} ({rep['layers']} layers): generated in {rep['wall_s']} s")
        for r in rep["prompts"]:
            print(f"  prompt {r['prompt_len']:6d}: divergence at {r['first_divergence']} (oracle margin "
                  f"{r['oracle_margin_there']}), oracle log-likelihood {r['oracle_loglik']}, {'ok' if r['ok'] else 'FAIL'}")
    return 0 if rep["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
