"""JSON / JSON-schema constrained decoding: byte machine acceptance and token masks."""
import json

import numpy as np
import pytest

from dgpp_b200.runtime import rt


def chk(schema, text):
    return rt.json_machine_check(json.dumps(schema) if schema is not None else "", text.encode())


def test_json_object_mode_accepts_exactly_objects():
    assert chk(None, '{"a": 1, "b": [true, null, {"c": "x\\n\\u00e9"}], "d": -1.5e+3}') == (True, True)
    assert chk(None, '{"a": 1') == (True, False)
    assert chk(None, '[1]')[0] is False                      # top level must be an object
    assert chk(None, '{"a": 01}')[0] is False                # leading zero
    assert chk(None, '{"a": 1,}')[0] is False                # trailing comma
    assert chk(None, '{"a": 1, "a": 2}')[0] is False         # duplicate key
    assert chk(None, '{"a": "\x01"}')[0] is False            # raw control character
    assert chk(None, '{      "a": 1}')[0] is False           # more than 4 blanks in a row
    assert chk(None, '{"a": tru')[0] is True and chk(None, '{"a": trx')[0] is False


SCHEMA = {"type": "object", "additionalProperties": False, "required": ["name", "age"],
          "properties": {"name": {"type": "string"}, "age": {"type": "integer"},
                         "tags": {"type": "array", "items": {"enum": ["a", "b", 3]}, "minItems": 1, "maxItems": 2},
                         "mode": {"const": "fast"}, "score": {"type": ["number", "null"]}}}


def test_schema_subset():
    assert chk(SCHEMA, '{"name": "x", "age": 3}') == (True, True)
    assert chk(SCHEMA, '{"age": 3, "name": "x", "tags": ["a", 3], "mode": "fast", "score": null}') == (True, True)
    assert chk(SCHEMA, '{"name": "x"}')[0] is False                       # required age missing at '}'
    assert chk(SCHEMA, '{"name": "x", "age": 3.5}')[0] is False           # integer
    assert chk(SCHEMA, '{"name": "x", "age": 3, "other": 1}')[0] is False  # additionalProperties false
    assert chk(SCHEMA, '{"name": "x", "age": 3, "tags": []}')[0] is False  # minItems
    assert chk(SCHEMA, '{"name": "x", "age": 3, "tags": ["a", "b", "a"]}')[0] is False   # maxItems
    assert chk(SCHEMA, '{"name": "x", "age": 3, "tags": ["c"]}')[0] is False  # enum
    assert chk(SCHEMA, '{"name": "x", "age": 3, "mode": "slow"}')[0] is False
    assert chk(SCHEMA, '{"name": "x", "age": 3, "score": 1e5}') == (True, True)
    assert chk(SCHEMA, '{"na') == (True, False) and chk(SCHEMA, '{"nb')[0] is False   # key prefixes are checked
    with pytest.raises(RuntimeError, match="anyOf"):
        chk({"anyOf": [{"type": "string"}]}, "1")
    with pytest.raises(RuntimeError, match="never be written"):
        chk({"type": "object", "required": ["x"], "additionalProperties": False, "properties": {}}, "{}")


def test_multiple_of_on_integers():
    sch = {"type": "object", "properties": {"n": {"type": "integer", "multipleOf": 25}}, "required": ["n"],
           "additionalProperties": False}
    for good in ('{"n": 0}', '{"n": 25}', '{"n": -1250}', '{"n": 100 }'):
        assert chk(sch, good) == (True, True), good
    for bad in ('{"n": 7}', '{"n": 26}', '{"n": -30}'):
        assert chk(sch, bad)[0] is False, bad
    assert chk(sch, '{"n": 12') == (True, False)             # may still become 125
    with pytest.raises(RuntimeError, match="multipleOf"):
        chk({"type": "number", "multipleOf": 0.5}, "1")


def test_token_masks_drive_a_valid_generation():
    # a toy vocabulary: single bytes plus a few multi-byte tokens and two specials
    vocab = [bytes([i]) for i in range(256)] + [b'{"', b'": ', b'", "', b'"}', b"true", b"null", b"name", b"age", b""]
    eos = len(vocab) - 1
    g = rt.JsonGrammar(json.dumps(SCHEMA), vocab, [eos])
    assert g.words() == (len(vocab) + 31) // 32

    def allowed():
        m = g.mask()
        return {i for i in range(len(vocab)) if (int(m[i >> 5]) >> (i & 31)) & 1}

    a0 = allowed()
    assert vocab.index(b'{"') in a0 and ord("{") in a0 and ord("[") not in a0 and eos not in a0
    # greedy walk: always take the allowed token that makes the text match a target document
    target = b'{"name": "bo", "age": 41}'
    text = b""
    steps = 0
    while text != target:
        al = allowed()
        cand = [i for i in al if i != eos and vocab[i] and target.startswith(text + vocab[i])]
        assert cand, (text, sorted(al)[:10])
        tok = max(cand, key=lambda i: len(vocab[i]))
        assert g.accept(tok)
        text += vocab[tok]
        steps += 1
    assert g.complete() and eos in allowed()
    assert steps < len(target)                       # multi-byte tokens were usable
    assert g.accept(eos)
    # a token that breaks the schema is refused
    g2 = rt.JsonGrammar(json.dumps(SCHEMA), vocab, [eos])
    assert not g2.accept(ord("["))
    # masks are cached per state: same object state -> identical mask
    g3 = rt.JsonGrammar("", vocab, [eos])
    assert np.array_equal(g3.mask(), g3.mask())


def _chk(schema, text):
    return rt.json_machine_check(json.dumps(schema), text.encode())


def test_string_lengths_patterns_and_formats():
    s = {"type": "string", "minLength": 2, "maxLength": 4}
    assert _chk(s, '"ab"') == (True, True) and _chk(s, '"a"') == (False, False) and _chk(s, '"abcd"') == (True, True)
    assert _chk(s, '"abcde') == (False, False) and _chk(s, '"a') == (True, False)
    assert _chk(s, '"héé"') == (True, True) and _chk(s, '"ééééé') == (False, False)      # code points, not bytes
    # anchored pattern: prefix viability is exact
    p = {"type": "string", "pattern": "^[A-Z]{2}-\\d{3}(x|yz)?$"}
    assert _chk(p, '"AB-123"') == (True, True) and _chk(p, '"AB-123yz"') == (True, True)
    assert _chk(p, '"AB-12') == (True, False) and _chk(p, '"AB-12"') == (False, False)
    assert _chk(p, '"Ab') == (False, False) and _chk(p, '"AB-123y"') == (False, False) and _chk(p, '"AB-123yzz') == (False, False)
    # unanchored pattern matches anywhere
    u = {"type": "string", "pattern": "ca+t"}
    assert _chk(u, '"a caaat!"') == (True, True) and _chk(u, '"dog"') == (False, False) and _chk(u, '"dog') == (True, False)
    # escapes are decoded before the pattern sees them; \\u is not accepted in a constrained body
    q = {"type": "string", "pattern": '^a"b\\nc$'}                     # regex: a " b newline c
    body = '"a' + chr(92) + '"b' + chr(92) + 'nc"'                    # JSON text: "a\"b\nc"
    assert _chk(q, body) == (True, True) and _chk(q, '"a"') == (False, False)
    assert _chk({"type": "string", "maxLength": 3}, '"' + chr(92) + 'u0041"') == (False, False)
    # formats
    assert _chk({"type": "string", "format": "date"}, '"2026-11-25"') == (True, True)
    assert _chk({"type": "string", "format": "date"}, '"2026/') == (False, False)
    assert _chk({"type": "string", "format": "uuid"}, '"123e4567-e89b-12d3-a456-426614174000"') == (True, True)
    assert _chk({"type": "string", "format": "date-time"}, '"2026-11-25T10:20:30.5+01:00"') == (True, True)
    assert _chk({"type": "string", "format": "hostname"}, '"anything"') == (True, True)          # unknown: annotation
    # inside an object, other properties are unaffected
    o = {"type": "object", "properties": {"id": {"type": "string", "pattern": "^\\d+$"}, "n": {"type": "string"}},
         "required": ["id"], "additionalProperties": False}
    assert _chk(o, '{"id": "42", "n": "free text"}') == (True, True) and _chk(o, '{"id": "4x') == (False, False)
    # outside the subset -> schema error at compile time
    for bad in ("(?=x)", "a{2,1}", "(", chr(92) + "1", "*a"):
        with pytest.raises(RuntimeError):
            rt.json_machine_check(json.dumps({"type": "string", "pattern": bad}), b'"')


def test_token_masks_follow_the_pattern():
    vocab = [bytes([i]) for i in range(256)] + [b"12", b"ab", b'"}', b""]
    eos = len(vocab) - 1
    schema = {"type": "object", "properties": {"zip": {"type": "string", "pattern": "^\\d{5}$"}}, "required": ["zip"],
              "additionalProperties": False}
    g = rt.JsonGrammar(json.dumps(schema), vocab, [eos])
    for b in b'{"zip": "12':
        assert g.accept(b)
    m = np.asarray(g.mask())
    allowed = {i for i in range(len(vocab)) if m[i >> 5] >> (i & 31) & 1}
    assert allowed == {ord(c) for c in "0123456789"} | {256}            # digits and the token "12"; not "ab", not '"'
    for b in b"345":
        assert g.accept(b)
    m = np.asarray(g.mask())
    allowed = {i for i in range(len(vocab)) if m[i >> 5] >> (i & 31) & 1}
    assert allowed == {ord('"'), 258}                                   # five digits written: only the closing quote
