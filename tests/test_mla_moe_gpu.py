"""MLA + MoE family on the GPU: the absorbed-attention kernel path (latent cache, sparse index, MoE block) against the
plain-attention PyTorch oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


@pytest.mark.parametrize("moe,index", [(False, False), (True, False), (False, True), (False, "fp8")])
def test_runner_matches_plain_attention_oracle(dev, moe, index):
    from dgpp_b200.models.mla_moe import MlaMoeConfig, MlaMoeModel, MlaMoeRunner
    from dgpp_b200.models.moe import MoEConfig
    from dgpp_b200.ops import core as ops

    cfg = MlaMoeConfig(layers=3, hidden=1024, heads=8, q_lora=256, kv_lora=128, nope=64, rope=32, v_dim=64, ffn=2048,
                       vocab=2048, dense_layers=1,
                       moe=MoEConfig(hidden=1024, experts=16, top_k=4, moe_ffn=512, shared_ffn=512) if moe else None,
                       index_heads=4 if index else 0, index_dim=128 if index == "fp8" else 64, index_topk=48,
                       index_key_fp8=index == "fp8")
    m = MlaMoeModel.random_init(cfg, dev, seed=3, std=0.04)
    r = MlaMoeRunner(m, max_rows=64, slots=2, max_seq_len=512, device=dev)
    assert (r.att.kidx[0].dtype == torch.uint8) == (index == "fp8") if index else True
    g = torch.Generator().manual_seed(2)
    a = torch.randint(0, cfg.vocab, (150,), generator=g).tolist()
    b = torch.randint(0, cfg.vocab, (37,), generator=g).tolist()
    la = r.prefill(0, a[:140], chunk=64).clone()
    lb = r.prefill(1, b[:30], chunk=16).clone()
    want_a = m.forward_reference(torch.tensor(a, device=dev))
    want_b = m.forward_reference(torch.tensor(b, device=dev))
    torch.cuda.synchronize()
    ops.check_status()

    def close(got, want, what):
        if moe:
            # the device router may break a near tie between two experts differently from the fp32 oracle router (its
            # inputs differ in the last bf16 bit): one swapped expert moves every logit a little, so the routed case
            # is judged by direction, the other cases element by element
            cos = torch.nn.functional.cosine_similarity(got.float(), want.float(), dim=0).item()
            assert cos >= 0.985, (what, cos)
            return
        err = (got - want).abs().max().item()
        lim = (0.12 if index else 0.06) * want.abs().max().item() + 0.02     # a top-k boundary may differ by one position
        assert err <= lim, (what, err, lim)

    close(la[-1], want_a[139], "prefill a")
    close(lb[-1], want_b[29], "prefill b")
    for s in range(4):                                   # batched decode, teacher-forced
        out = r.decode([0, 1], [a[140 + s], b[30 + s]])
        close(out[0], want_a[140 + s], f"decode a {s}")
        close(out[1], want_b[30 + s], f"decode b {s}")
    assert r.lengths == [144, 34]


def test_yarn_scaled_rotary_and_shared_or_cloned_prefixes(dev):
    """YaRN factor 4 over a short original context (the oracle and the kernels read the same frequency table and
    softmax scale); a second slot that reads the first slot's prefix blocks, or a copy of them, decodes to the same
    logits as the first slot does."""
    from dgpp_b200.models.mla_moe import MlaMoeConfig, MlaMoeModel, MlaMoeRunner, softmax_scale
    from dgpp_b200.ops import core as ops

    cfg = MlaMoeConfig(layers=2, hidden=1024, heads=8, q_lora=256, kv_lora=128, nope=64, rope=32, v_dim=64, ffn=2048,
                       vocab=2048, dense_layers=2, index_heads=4, index_dim=128, index_topk=48, yarn_factor=4.0,
                       yarn_orig_ctx=64)
    assert softmax_scale(cfg) > 1.0 / (cfg.nope + cfg.rope) ** 0.5
    m = MlaMoeModel.random_init(cfg, dev, seed=3, std=0.04)
    g = torch.Generator().manual_seed(4)
    toks = torch.randint(0, cfg.vocab, (200,), generator=g).tolist()
    want = m.forward_reference(torch.tensor(toks, device=dev))
    for shared in (False, True):
        r = MlaMoeRunner(m, max_rows=64, slots=3, max_seq_len=512, device=dev, shared_tail_blocks=2 if shared else 0)
        last = r.prefill(0, toks[:192], chunk=64)
        err = (last[-1] - want[191]).abs().max().item()
        assert err <= 0.12 * want[191].abs().max().item() + 0.02, err
        for s in (1, 2):
            if shared:
                r.att.share_prefix(s, 192)
            else:
                r.att.clone_prefix(s, 192)
            r.lengths[s] = 192
        out = r.decode([0, 1, 2], [toks[192]] * 3).clone()
        assert torch.equal(out[0], out[1]) and torch.equal(out[0], out[2]), shared
        out2 = r.decode([2, 0], [toks[193], toks[193]])
        assert torch.equal(out2[0], out2[1])
        assert (out2[0] - want[193]).abs().max().item() <= 0.12 * want[193].abs().max().item() + 0.02
    torch.cuda.synchronize()
    ops.check_status()


@pytest.mark.parametrize("moe", [False, True])
def test_decode_width_block_scaled_linears(dev, moe):
    """NVFP4 weights: decode-width passes take the block-scaled path (norm kernels emit three-term NVFP4 rows, packed
    weights stream as stored); logits stay within the oracle's tolerance and close to the converter path's."""
    from dgpp_b200.models.mla_moe import MlaMoeConfig, MlaMoeModel, MlaMoeRunner
    from dgpp_b200.models.moe import MoEConfig
    from dgpp_b200.ops import core as ops

    cfg = MlaMoeConfig(layers=3, hidden=1024, heads=8, q_lora=256, kv_lora=128, nope=64, rope=32, v_dim=64, ffn=2048,
                       vocab=2048, dense_layers=1, index_heads=4, index_dim=128, index_topk=48, index_key_fp8=True,
                       moe=MoEConfig(hidden=1024, experts=16, top_k=4, moe_ffn=512, shared_ffn=512) if moe else None)
    m = MlaMoeModel.random_init(cfg, dev, seed=3, std=0.04, fmt="nvfp4")
    assert m.layers[0].q_a.fmt == "nvfp4" and m.layers[0].o.fmt == "nvfp4"
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, cfg.vocab, (90,), generator=g).tolist()
    want = m.forward_reference(torch.tensor(toks, device=dev))
    outs = {}
    for fp4 in (True, False):
        r = MlaMoeRunner(m, max_rows=64, slots=2, max_seq_len=256, device=dev)
        r.decode_fp4 = fp4
        r.prefill(0, toks[:80], chunk=64)
        r.prefill(1, toks[:70], chunk=64)
        seq = []
        for s in range(6):
            out = r.decode([0, 1] if s < 3 else [0], [toks[80 + s], toks[70 + s]] if s < 3 else [toks[80 + s]])
            seq.append(out[0].clone())
        outs[fp4] = seq
        if fp4:
            assert r.att.dq.bufs, "the block-scaled path did not run"
    torch.cuda.synchronize()
    ops.check_status()
    for s in range(6):
        ref_row = want[80 + s]
        for fp4 in (True, False):
            got = outs[fp4][s]
            if moe:
                cos = torch.nn.functional.cosine_similarity(got.float(), ref_row.float(), dim=0).item()
                assert cos >= 0.98, (fp4, s, cos)
            else:
                err = (got - ref_row).abs().max().item()
                assert err <= 0.12 * ref_row.abs().max().item() + 0.03, (fp4, s, err)
