"""Hashed n-gram memory on the GPU: lookup and gate kernels against their oracles, and the sites inside the stream
family's runner (chunked prefill, graph decode, reset)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def test_lookup_and_gate_kernels(dev):
    from dgpp_b200.models.engram import Engram, EngramConfig
    from dgpp_b200.ops import core as ops
    from dgpp_b200.ops import reference as ref

    cfg = EngramConfig(max_ngram=4, heads=3, head_dim=64, bucket=2000)
    e = Engram.random_init(cfg, [0], 1000, 4, 512, dev, seed=5)
    L = e.layers[0]
    L.multipliers = torch.tensor([0x7123456789ABCDE1, 0x6FEDCBA987654321, 0x5555555555555555, 0x7777777777777771],
                                 dtype=torch.int64, device=dev)                       # products that wrap
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, 1000, (77,), generator=g, dtype=torch.int32)
    prev = torch.tensor(e.prev_rows(toks.tolist(), []), dtype=torch.int32, device=dev)
    toks = toks.to(dev)
    ids = torch.empty(77, cfg.slots, dtype=torch.int32, device=dev)
    out = ops.engram_embed(toks, prev, e.token_map, L.multipliers, L.primes, L.offsets, L.table, L.table_sf, e.pad_class, ids=ids)
    want_ids = ref.engram_ids(toks, prev, e.token_map, L.multipliers, L.primes, L.offsets, e.pad_class)
    want = ref.engram_embed(toks, prev, e.token_map, L.multipliers, L.primes, L.offsets, L.table, L.table_sf, e.pad_class)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(ids.long(), want_ids)
    assert torch.equal(out, want)                                                    # the decode is exact
    gd = torch.Generator(device=dev).manual_seed(2)
    x = torch.randn(77, 4, 512, device=dev, generator=gd).to(BF)
    kv = ops.linear(out, L.wkv)
    want_x = ref.engram_gate(x, kv, L.q_weight, L.k_weight, 1e-6)
    got_x = ops.engram_gate(x.clone(), kv, L.q_weight, L.k_weight, 1e-6)
    torch.cuda.synchronize()
    ops.check_status()
    assert (got_x.float() - want_x.float()).abs().max().item() <= 0.02 * want_x.float().abs().max().item()
    assert (got_x.float() - x.float()).abs().max().item() > 1e-2


def test_stream_family_runner_with_memory_sites(dev):
    from dgpp_b200.models.engram import EngramConfig
    from dgpp_b200.models.glm_flash import GlmFlashConfig, GlmFlashModel, GlmFlashRunner
    from dgpp_b200.ops import core as ops

    cfg = GlmFlashConfig(layers=4, hidden=1024, vocab=2048, mla_every=2, streams=4, k_heads=2, v_heads=4, dk=128, dv=128,
                         heads=8, q_lora=256, kv_lora=128, nope=64, rope=32, v_dim=64, ffn=2048,
                         engram=EngramConfig(max_ngram=4, heads=2, head_dim=64, bucket=3000), engram_layers=(0, 2))
    m = GlmFlashModel.random_init(cfg, dev, seed=3, std=0.04)
    r = GlmFlashRunner(m, max_rows=64, slots=3, max_seq_len=512, device=dev)
    g = torch.Generator().manual_seed(2)
    a = torch.randint(0, cfg.vocab, (110,), generator=g).tolist()
    b = torch.randint(0, cfg.vocab, (37,), generator=g).tolist()
    la = r.prefill(2, a[:100], chunk=64).clone()
    lb = r.prefill(0, b[:30], chunk=16).clone()
    want_a = m.forward_reference(torch.tensor(a, device=dev))
    want_b = m.forward_reference(torch.tensor(b, device=dev))
    torch.cuda.synchronize()
    ops.check_status()

    def close(got, want, what):
        err = (got - want).abs().max().item()
        lim = 0.06 * want.abs().max().item() + 0.02
        assert err <= lim, (what, err, lim)

    close(la[-1], want_a[99], "prefill a")
    close(lb[-1], want_b[29], "prefill b")
    for s in range(4):
        out = r.decode([2, 0], [a[100 + s], b[30 + s]])
        close(out[0], want_a[100 + s], f"decode a {s}")
        close(out[1], want_b[30 + s], f"decode b {s}")
    assert r.history[2] == a[101:104] and r.history[0] == b[31:34]
    torch.cuda.synchronize()
    ops.check_status()
    r.reset(0)
    assert r.history[0] == [] and torch.equal(r.prefill(0, b[:30], chunk=16), lb)
