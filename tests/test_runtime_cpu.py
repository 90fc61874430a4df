"""Host runtime (native C++): paged blocks, prefix cache, scheduler on the fake engine, tokenizer, chat template."""
import json
import random
import unicodedata

import pytest

from dgpp_b200.runtime import rt


def _trace(seed=0, n=64, vocab=4096, shared_len=256):
    rng = random.Random(seed)
    shared = [rng.randrange(vocab) for _ in range(shared_len)]
    reqs = {}
    for i in range(n):
        ln = rng.randint(16, 512)
        if i % 2 == 0:
            p = shared + [rng.randrange(vocab) for _ in range(max(1, ln - shared_len))]
        else:
            p = [rng.randrange(vocab) for _ in range(ln)]
        reqs[f"r{i}"] = p
    return reqs


def _run(reqs, slots=4, blocks=200, policy=None, tokens_per_step=1, prefix=True, budget=None, group=1):
    eng = rt.FakeEngine(slots=slots, block_tokens=16, blocks=blocks, max_context=1024, vocab=4096,
                        tokens_per_step=tokens_per_step)
    cfg = rt.SchedulerConfig()
    cfg.prefix_cache = prefix
    if policy is not None:
        cfg.policy = policy
    if budget is not None:
        cfg.prefill_budget_idle = cfg.prefill_budget_busy = cfg.prefill_chunk = budget
    cfg.prefill_group_max = group
    s = rt.Scheduler(eng, cfg)
    for rid, p in reqs.items():
        s.submit(rid, p, 32)
    s.run(200000)
    out, retire = {}, {}
    for kind, rid, a, b in s.events():
        if kind == "token":
            out.setdefault(rid, []).append(a)
        elif kind.startswith("retire"):
            retire[rid] = (kind, b)
    return s, eng, out, retire


def test_paged_block_table():
    t = rt.PagedBlockTable(3)
    a, b, c = t.alloc(), t.alloc(), t.alloc()
    assert sorted([a, b, c]) == [0, 1, 2] and t.alloc() == -1
    t.retain(b)
    t.release(b)
    assert t.refcount(b) == 1 and t.free_count() == 0
    g = t.generation(b)
    t.release(b)
    assert t.free_count() == 1 and t.alloc() == b and t.generation(b) == g + 1
    with pytest.raises(Exception):
        t.release(99)


def test_scheduler_trace_is_exact_and_uses_prefix_cache():
    reqs = _trace()
    s, eng, out, retire = _run(reqs)
    for rid, p in reqs.items():
        assert out[rid] == rt.FakeEngine.expected(p, 32, 4096), rid
        assert retire[rid][0] == "retire:length"
    m = s.meters()
    assert m["admitted"] == 64 and m["retired"] == 64
    assert m["prefix_hit_tokens"] > 0 and m["prefix_hits"] > 0
    # the engine never re-prefilled cached positions
    assert m["prefill_tokens"] == sum(len(p) for p in reqs.values()) - m["prefix_hit_tokens"]


def test_scheduler_is_deterministic_and_scheduling_invariant():
    reqs = _trace(seed=3)
    s1, _, out1, _ = _run(reqs)
    s2, _, out2, _ = _run(reqs)
    assert out1 == out2 and s1.op_digest() == s2.op_digest() and s1.prefix_digest() == s2.prefix_digest()
    # different slot counts, budgets, cache off, multi-token steps: same tokens per request
    for kw in (dict(slots=1), dict(slots=8, blocks=400), dict(prefix=False), dict(budget=48), dict(tokens_per_step=3),
               dict(group=4), dict(group=8, slots=8, blocks=400, budget=96), dict(group=3, prefix=False)):
        _, _, out3, _ = _run(reqs, **kw)
        for rid in reqs:
            assert out3[rid][:32] == out1[rid], (kw, rid)


def test_group_prefill_packs_readers_into_fewer_engine_calls():
    """Readers of a tick advance together: the engine sees fewer prefill calls for the same prompt tokens, short prompts
    finish next to a long one instead of behind it, tokens per request do not change."""
    rng = random.Random(5)
    reqs = {f"r{i}": [rng.randrange(4096) for _ in range(n)] for i, n in enumerate((400, 20, 25, 30, 18, 22))}
    s1, _, out1, _ = _run(reqs, slots=6, prefix=False, budget=128)
    s4, _, out4, _ = _run(reqs, slots=6, prefix=False, budget=128, group=6)
    assert out1 == out4
    m1, m4 = s1.meters(), s4.meters()
    assert m4["prefill_tokens"] == m1["prefill_tokens"] and m4["prefill_calls"] < m1["prefill_calls"]

    # what the engine is handed: a Python engine (the CPU oracle model) records its group calls
    import torch
    from dgpp_b200.engine.adapters import ReferenceEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel
    from dgpp_b200.ops import reference as ref

    class Recorder(ReferenceEngine):
        calls = []

        def prefill_group(self, pieces):
            Recorder.calls.append([(s, len(t), p, l) for s, t, p, l in pieces])
            return [self.prefill(s, t, p, l) for s, t, p, l in pieces]

    m = DenseModel.random_init(DenseConfig.plumbing_fp32(), device="cpu", seed=0, std=0.02)
    short = {rid: p[:60] if len(p) > 60 else p for rid, p in reqs.items()}
    short["r0"] = reqs["r0"][:200]

    def run(group):
        Recorder.calls = []
        with ref.activation_dtype(torch.float32):
            eng = Recorder(m, slots=6, num_blocks=128, block_tokens=16, max_context=256)
            cfg = rt.SchedulerConfig()
            cfg.prefix_cache = False
            cfg.prefill_budget_idle = cfg.prefill_budget_busy = cfg.prefill_chunk = 128
            cfg.prefill_group_max = group
            s = rt.Scheduler(eng, cfg)
            for rid, p in short.items():
                s.submit(rid, p, 3)
            s.run(10000)
        return {rid: [a for kind, r, a, b in s.events() if kind == "token" and r == rid] for rid in short}

    base = run(1)
    assert not Recorder.calls
    grouped = run(6)
    assert grouped == base
    first = Recorder.calls[0]
    assert len(first) == 6 and sum(n for _, n, _, _ in first) <= 128
    assert sum(last for _, n, _, last in first[1:]) >= 4 and not first[0][3]    # the short prompts finish in call one
    assert first[0][1] >= 128 // 6                                              # the long reader still got its share


def test_grow_on_demand_sheds_youngest_and_recovers():
    reqs = {f"r{i}": [i + 1] * 40 for i in range(6)}
    s, eng, out, retire = _run(reqs, slots=4, blocks=14, policy=rt.AdmissionPolicy.GrowOnDemand, prefix=False)
    for rid, p in reqs.items():
        assert out[rid] == rt.FakeEngine.expected(p, 32, 4096)
    assert s.meters()["shed"] >= 1
    assert eng.free_blocks() == eng.total_blocks()


def test_cancel_and_eos():
    eng = rt.FakeEngine(slots=2, block_tokens=16, blocks=64, max_context=512, vocab=50)
    s = rt.Scheduler(eng, rt.SchedulerConfig())
    p = list(range(20))
    exp = rt.FakeEngine.expected(p, 64, 50)
    eos = exp[5]
    first_eos = exp.index(eos)
    s.submit("a", p, 64, eos_ids=[eos])
    s.submit("b", p, 64)
    s.submit("c", p, 64)
    for _ in range(3):
        s.tick()
    s.cancel("b")
    s.cancel("c")
    s.run()
    ev = s.events()
    toks = [a for k, rid, a, b in ev if k == "token" and rid == "a"]
    assert toks == exp[:first_eos]
    kinds = {rid: k for k, rid, a, b in ev if k.startswith("retire")}
    assert kinds["a"] == "retire:stop" and kinds["b"] == "retire:cancelled" and kinds["c"] == "retire:cancelled"


def test_chain_hash_is_prefix_sensitive():
    h1 = rt.chain_hash(rt.FNV_SEED, list(range(16)))
    h2 = rt.chain_hash(rt.FNV_SEED, list(range(1, 17)))
    assert h1 != h2 and rt.chain_hash(h1, list(range(16))) != h1


# ------------------------------------------------------------------ text stack
MERGES = [(b"t", b"h"), (b"th", b"e"), (b" ", b"th"), (b" th", b"e"), (b"i", b"n"), (b"e", b"r"), (b" ", b"a"),
          (b" a", b"n"), (b" an", b"d"), (b"o", b"r"), (b"l", b"l"), (b"1", b"2")]
TEXTS = ["the cat and the other thing's 123 héllo  \n\n world !", "  multiple   spaces\tand\ttabs  ",
         "naïve café 北京 12345 'll've", "a\n\n\nb   \n c", "Hello, World!! 2024-01-02\r\n\r\nNew  line's HERE'S\n",
         "x=1;y=22;zzz=333", "", " ", "\n", "end with space ", "emoji 😀😀 ok", "١٢٣ arabic digits", "don't I'LL we'Ve"]


def test_tokenizer_roundtrip_and_special_tokens():
    tok = rt.Tokenizer.byte_level(MERGES, [("<|eot|>", 300, True)], rt.SplitPattern.Gpt2)
    for t in TEXTS:
        assert tok.decode(tok.encode(t)).decode() == t
    ids = tok.encode("hi<|eot|>there")
    assert 300 in ids and tok.is_special(300)
    assert 300 not in tok.encode("hi<|eot|>there", allow_special=False)
    assert tok.decode(ids, skip_special=True).decode() == "hithere"
    assert tok.token_to_id("the") == tok.encode("the")[0]


@pytest.mark.parametrize("pattern,regex", [
    ("Gpt2", None),
    ("Qwen2", r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"),
    ("Cl100k", r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"),
])
def test_tokenizer_matches_hf_tokenizers(pattern, regex):
    hf = pytest.importorskip("tokenizers")
    from tokenizers import Regex, models, pre_tokenizers

    def mapb(b):
        bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
        cs, n = bs[:], 0
        for x in range(256):
            if x not in bs:
                bs.append(x)
                cs.append(256 + n)
                n += 1
        d = dict(zip(bs, [chr(c) for c in cs]))
        return "".join(d[x] for x in b)

    vocab = {mapb(bytes([i])): i for i in range(256)}
    ms = []
    for a, b in MERGES:
        ms.append((mapb(a), mapb(b)))
        vocab.setdefault(mapb(a) + mapb(b), len(vocab))
    ht = hf.Tokenizer(models.BPE(vocab=vocab, merges=ms))
    if regex is None:
        ht.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    else:
        ht.pre_tokenizer = pre_tokenizers.Sequence([
            pre_tokenizers.Split(Regex(regex), behavior="isolated"),
            pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    mine = rt.Tokenizer.byte_level(MERGES, [], getattr(rt.SplitPattern, pattern))
    for t in TEXTS:
        assert ht.encode(t).ids == mine.encode(t), t


def test_tokenizer_json_loader_and_stream_decoder():
    hf = pytest.importorskip("tokenizers")
    from tokenizers import models, pre_tokenizers, decoders

    vocab = {"a": 0, "b": 1, "ab": 2, "Ġ": 3, "Ġab": 4, "c": 5}
    ht = hf.Tokenizer(models.BPE(vocab=vocab, merges=[("a", "b"), ("Ġ", "ab")]))
    ht.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    ht.add_special_tokens(["<s>"])
    tok = rt.Tokenizer.from_json(ht.to_str())
    assert tok.encode("ab ab c<s>") == ht.encode("ab ab c<s>").ids
    t2 = rt.Tokenizer.byte_level(MERGES, [], rt.SplitPattern.Gpt2)
    sd = rt.StreamDecoder(t2)
    pieces = [sd.push(i) for i in t2.encode("héllo 北京😀")]
    for p in pieces:
        p.decode("utf-8")  # every piece is valid UTF-8 on its own
    assert (b"".join(pieces) + sd.flush()).decode() == "héllo 北京😀"


def test_nfc_matches_unicodedata():
    for t in ["école", "각", "Å", "Ậ", "plain ascii", "q̣̇", "가각"]:
        assert rt.Tokenizer.normalize_nfc(t) == unicodedata.normalize("NFC", t), repr(t)


CHATML = """{%- for message in messages %}
    {%- if loop.first and message['role'] != 'system' %}
        {{- '<|im_start|>system\\nYou are a helpful assistant.<|im_end|>\\n' }}
    {%- endif %}
    {{- '<|im_start|>' + message['role'] + '\\n' + message['content'] | trim + '<|im_end|>' + '\\n' }}
{%- endfor %}
{%- if add_generation_prompt %}
    {{- '<|im_start|>assistant\\n' }}
{%- endif %}"""

FEATURES = """{% set ns = namespace(n=0) %}{% for m in messages if m.role != 'system' %}{% set ns.n = ns.n + 1 %}[{{ loop.index }}/{{ loop.length }}:{{ m.role|upper }}:{{ m.content|length }}]{% else %}none{% endfor %} total={{ ns.n }} {{ 'a,b'.split(',') | join('-') }} {{ x is defined }} {{ 7 // 2 }} {{ -7 % 3 }} {{ 'yes' if messages else 'no' }} {{ messages[-1].content[::-1] }} {{ messages | map(attribute='role') | list | length }}
{% macro greet(name, punct='!') %}Hello {{ name }}{{ punct }}{% endmacro %}{{ greet('Bob') }} {{ greet('Al', punct='?') }}
{%- if tools is defined and tools %} T={{ tools | length }}{% endif %} {{ messages | selectattr('role', 'equalto', 'user') | list | length }} {{ [1, 2] + [3] }} {{ {'k': 1}.get('z', 'dflt') }}"""


@pytest.mark.parametrize("tpl", [CHATML, FEATURES])
def test_chat_template_matches_jinja2(tpl):
    jinja2 = pytest.importorskip("jinja2")
    ctx = {"messages": [{"role": "user", "content": " hi there "}, {"role": "assistant", "content": "yo"}],
           "add_generation_prompt": True, "tools": [{"type": "function"}]}
    env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True)
    want = env.from_string(tpl).render(**ctx)
    assert rt.ChatTemplate(tpl).render_json(json.dumps(ctx)) == want


def test_chat_template_tojson_errors_and_limits():
    t = rt.ChatTemplate("{{ tools | tojson }}|{{ tools | tojson(indent=2) }}")
    out = t.render_json(json.dumps({"tools": [{"b": 1, "a": "é"}]}))
    assert out.startswith('[{"b": 1, "a": "é"}]|[\n  {\n    "b": 1')
    with pytest.raises(Exception, match="raised: nope"):
        rt.ChatTemplate("{{ raise_exception('nope') }}").render_json("{}")
    with pytest.raises(Exception, match="byte"):
        rt.ChatTemplate("{% if x %}unterminated")
    with pytest.raises(Exception, match="limit|too large"):
        rt.ChatTemplate("{% for i in range(100000) %}{% for j in range(100000) %}x{% endfor %}{% endfor %}",
                        max_output_bytes=1 << 20, max_loop_iterations=10000).render_json("{}")


def test_json_parser_strictness():
    assert json.loads(rt.json_roundtrip('{"a": [1, 2.5, "x\\u00e9\\ud83d\\ude00", null, true]}')) == \
        {"a": [1, 2.5, "xé😀", None, True]}
    with pytest.raises(Exception, match="duplicate"):
        rt.json_roundtrip('{"a": 1, "a": 2}', reject_duplicates=True)
    for bad in ['{"a": }', '[1,]', '{"a" 1}', '"\\x"', '01', '[1] x']:
        with pytest.raises(Exception):
            rt.json_roundtrip(bad)


def test_engine_can_shorten_a_prefix_hit():
    """An engine that can only resume at some block boundaries (recurrent state snapshots) trims the matched chain."""
    class Eng(rt.SchedulerEngine):
        def __init__(self):
            super().__init__()
            self.t = rt.PagedBlockTable(64)
            self.blocks = {}
            self.attached = []
            self.prefilled = []
        def max_concurrent(self): return 2
        def block_tokens(self): return 16
        def total_blocks(self): return 64
        def free_blocks(self): return self.t.free_count()
        def max_context(self): return 512
        def reserve(self, slot, tokens):
            cur = self.blocks.setdefault(slot, [])
            while len(cur) * 16 < tokens:
                cur.append(self.t.alloc())
            return True
        def usable_prefix(self, blocks): return len(blocks) // 4 * 4      # snapshots every 4 blocks
        def attach_prefix(self, slot, blocks):
            self.attached.append(len(blocks))
            for b in blocks:
                self.t.retain(b)
            self.blocks[slot] = list(blocks)
        def prefill(self, slot, tokens, pos, last):
            self.prefilled.append((pos, len(tokens)))
            return 7 if last else -1
        def step_batch(self, slots): return [[7] for _ in slots]
        def slot_blocks(self, slot): return list(self.blocks.get(slot, []))
        def retain_block(self, b): self.t.retain(b)
        def release_block(self, b): self.t.release(b)
        def block_refcount(self, b): return self.t.refcount(b)
        def close(self, slot):
            for b in self.blocks.pop(slot, []):
                self.t.release(b)

    eng = Eng()
    cfg = rt.SchedulerConfig()
    cfg.prefix_min_tokens = 16
    s = rt.Scheduler(eng, cfg)
    prompt = list(range(100, 100 + 16 * 7 + 5))          # 7 full blocks + 5 tokens
    s.submit("a", prompt, 2)
    s.run(10000)
    s.submit("b", prompt, 2)
    s.run(10000)
    assert eng.attached == [4]                            # 7 blocks matched, the engine resumes at block 4
    assert s.meters()["prefix_hit_tokens"] == 64
    assert (64, len(prompt) - 64) in eng.prefilled or sum(n for p, n in eng.prefilled if p >= 64) >= len(prompt) - 64


def test_mixed_passes_carry_decoders_with_the_readers_chunk():
    """With mixed passes on, a reader's chunk and the decode step of everybody decoding are one engine call: same
    tokens as without, fewer engine calls, and decoders advance in every tick a reader is prefilling."""
    reqs = _trace(n=24, seed=5)

    def run(mixed, engine_mixed=True):
        eng = rt.FakeEngine(slots=4, block_tokens=16, blocks=200, max_context=1024, vocab=4096)
        eng.mixed = engine_mixed
        cfg = rt.SchedulerConfig()
        cfg.prefix_cache = False
        cfg.prefill_budget_idle = cfg.prefill_budget_busy = cfg.prefill_chunk = 24
        cfg.mixed_pass = mixed
        s = rt.Scheduler(eng, cfg)
        for rid, p in reqs.items():
            s.submit(rid, p, 32)
        s.run(200000)
        out = {}
        for kind, rid, a, b in s.events():
            if kind == "token":
                out.setdefault(rid, []).append(a)
        return s.meters(), eng, out

    m0, e0, out0 = run(False)
    m1, e1, out1 = run(True)
    for rid, p in reqs.items():
        assert out0[rid] == out1[rid] == rt.FakeEngine.expected(p, 32, 4096), rid
    assert m0["mixed_passes"] == 0 and m1["mixed_passes"] > 0 and e1.mixed_calls == m1["mixed_passes"]
    calls0 = e0.prefill_calls + e0.decode_passes
    calls1 = e1.prefill_calls + e1.decode_passes + e1.mixed_calls
    # every mixed pass saves a call, give or take the few ticks whose plan shifts (a reader that finishes inside a mixed
    # pass takes its first decode step one tick later)
    assert calls1 < calls0 and abs((calls0 - calls1) - m1["mixed_passes"]) <= 0.05 * m1["mixed_passes"]
    assert m1["prefill_tokens"] == m0["prefill_tokens"] == sum(len(p) for p in reqs.values())
    # an engine without a mixed pass: the scheduler falls back to the two calls, nothing changes
    m2, e2, out2 = run(True, engine_mixed=False)
    assert out2 == out0 and m2["mixed_passes"] == 0 and e2.prefill_calls == e0.prefill_calls
