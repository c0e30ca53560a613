"""Constrained JSON output on the host: the incremental automaton behind arcs_jcon_* against
(1) the known answers of the reference's own test (tests/test_api_compat.cpp:17-56), which pin it
without the reference tree, and (2) jcon::Checker itself (oracle/_ref, when built) on every prefix
of valid and damaged documents, and token by token over a synthetic vocabulary: the table's mask
bit t must equal check(text + piece(t)) != FAIL, which is what tools/server_chat.h:553-557 asks
per candidate. No GPU needed."""
import ctypes as C
import json

import numpy as np
import pytest

import orc
from arcinfer_b200 import jcon

F, P, D = jcon.FAIL, jcon.PARTIAL, jcon.DONE

SCHEMA_PERSON = (
    '{"type":"object","properties":{"name":{"type":"string"},"age":{"type":"integer"},'
    '"tags":{"type":"array","items":{"enum":["a","bb"]},"maxItems":2},"kind":{"anyOf":[{"type":"null"},{"const":"x"}]}},'
    '"required":["name","age"]}'
)
SCHEMA_REF = (
    '{"$defs":{"P":{"type":"object","properties":{"x":{"type":"number"}},"required":["x"]}},'
    '"type":"array","items":{"$ref":"#/$defs/P"}}'
)
# the reference's known answers: (schema, object_only, text, result)
KNOWN = [
    ("{}", True, "", P),
    ("{}", True, "  {", P),
    ("{}", True, '{"a": [1, 2, {"b": null}], "c": "x\\ny"}', D),
    ("{}", True, "[1]", F),
    ("{}", True, '{"a": 1}}', F),
    ("{}", True, '{"a": 01}', F),
    ("{}", True, '{"a": tru', P),
    ("{}", True, '{"a": trux', F),
    ("{}", True, '{"a": "\\u00', P),
    ("{}", True, '{"a": "\\q"}', F),
    ("{}", True, '{"a":1}            ', F),
    (SCHEMA_PERSON, False, '{"name": "Ann", "age": 30}', D),
    (SCHEMA_PERSON, False, '{"name": "Ann"}', F),
    (SCHEMA_PERSON, False, '{"na', P),
    (SCHEMA_PERSON, False, '{"nx', F),
    (SCHEMA_PERSON, False, '{"name": "A", "name": "B"', F),
    (SCHEMA_PERSON, False, '{"age": 3.5', F),
    (SCHEMA_PERSON, False, '{"age": "3"', F),
    (SCHEMA_PERSON, False, '{"name":"a","age":1,"tags":["b', P),
    (SCHEMA_PERSON, False, '{"name":"a","age":1,"tags":["c', F),
    (SCHEMA_PERSON, False, '{"name":"a","age":1,"tags":["a","bb","a"', F),
    (SCHEMA_PERSON, False, '{"name":"a","age":1,"kind":null}', D),
    (SCHEMA_PERSON, False, '{"name":"a","age":1,"kind":"x"}', D),
    (SCHEMA_PERSON, False, '{"name":"a","age":1,"kind":"y"', F),
    (SCHEMA_REF, False, '[{"x": -1.5e3}, {"x": 2}]', D),
    (SCHEMA_REF, False, '[{"y": 1}]', F),
]

EMPTY_VOCAB = (np.zeros(1, np.uint32), np.zeros(0, np.uint8))


def test_known_answers_of_the_reference_test():
    made = {}
    for schema, obj, text, want in KNOWN:
        jc = made.setdefault((schema, obj), jcon.JsonConstraint(schema, obj, *EMPTY_VOCAB))
        assert jc.check(text) == want, (schema[:40], text)


SCHEMAS = [
    ("{}", True),
    ("{}", False),
    (SCHEMA_PERSON, False),
    (SCHEMA_REF, False),
    ('{"type":"object","properties":{"id":{"type":"integer"},"ok":{"type":"boolean"},"note":{"type":["string","null"]},'
     '"pos":{"type":"array","items":{"type":"number"},"minItems":2,"maxItems":3}},"required":["id"],'
     '"additionalProperties":{"type":"string"}}', False),
    ('{"type":"object","properties":{"mode":{"enum":["fast","slow",3,null,true]},"inner":{"type":"object",'
     '"properties":{"k":{"const":{"a":[1,2]}}},"additionalProperties":true}},"additionalProperties":false}', False),
    ('{"type":"array","items":{"anyOf":[{"type":"string"},{"type":"integer"},{"type":"array","items":{"type":"boolean"}}]},"minItems":1}', False),
    ('{"definitions":{"N":{"type":"object","properties":{"v":{"type":"integer"},"next":{"anyOf":[{"type":"null"},{"$ref":"#/definitions/N"}]}},'
     '"required":["v","next"]}},"$ref":"#/definitions/N"}', False),
]

DOCS = {
    0: ['{"a": [1, 2, {"b": null}], "c": "x\\ny"}', '{ "k" : -0.5e+10 , "ü": [ ] , "z":{}}', '{"a":{"a":{"a":[[[true,false]]]}}} '],
    1: ['[1, "two", {"three": 3.0}]', ' "just a string \\u00e9 \\" "', "-12.5E-3 ", "null", "[[[[[[1]]]]]]"],
    2: ['{"name": "Ann", "age": 30}', '{"age":1,"name":"a","tags":["a","bb"],"kind":null}', '{"name":"a","age":-7,"kind":"x","tags":[]}'],
    3: ['[{"x": -1.5e3}, {"x": 2}]', "[]", '[ {"x":0} ]'],
    4: ['{"id": 5, "ok": true, "note": null, "pos": [1, 2.5], "extra": "s", "more": "t"}', '{"x":"y","id":0,"pos":[1,2,3],"note":"n"}'],
    5: ['{"mode":"fast","inner":{"k":{"a":[1,2]},"z":[1,{"q":null}]}}', '{"mode":3}', '{"mode":null,"inner":{}}', '{"inner":{"free":1},"mode":true}'],
    6: ['["a", 12, [true, false], "b"]', "[[]]", '[ -3 , "x" ]'],
    7: ['{"v":1,"next":{"v":2,"next":{"v":3,"next":null}}}', '{"next":null,"v":0}'],
}


def damaged(doc, rng, n):
    """n variants of doc with one byte replaced, inserted or removed."""
    pool = b'{}[]:,"\\ \n0123456789-+.eEtruefalsn' + b"axyzk\xc3\xbc\x01"
    b = doc.encode()
    out = []
    for _ in range(n):
        i = int(rng.integers(0, len(b) + 1))
        c = bytes([pool[int(rng.integers(0, len(pool)))]])
        kind = int(rng.integers(0, 3))
        out.append(b[:i] + c + b[i:] if kind == 0 else b[:i] + c + b[i + 1:] if kind == 1 else b[:i] + b[i + 1:])
    return out


def ref_check(schema, obj, text):
    return orc.ref.ref_jcon_check(schema.encode(), int(obj), text, len(text))


needs_ref = pytest.mark.skipif(orc.ref is None, reason="oracle/_ref/libarcs_ref.so not built (needs the reference tree)")


@needs_ref
def test_every_prefix_against_the_reference_checker():
    rng = np.random.default_rng(11)
    n = 0
    for si, (schema, obj) in enumerate(SCHEMAS):
        jc = jcon.JsonConstraint(schema, obj, *EMPTY_VOCAB)
        for doc in DOCS[si]:
            for text in [doc.encode()] + damaged(doc, rng, 40):
                for cut in range(len(text) + 1):
                    got, want = jc.check(text[:cut]), ref_check(schema, obj, text[:cut])
                    assert got == want, (si, text[:cut], got, want)
                    n += 1
                    if want == F:
                        break  # (longer prefixes fail too; one past the first failure is checked below)
                if cut < len(text):
                    assert jc.check(text) == ref_check(schema, obj, text) == F
    assert n > 5000


def json_vocab(rng, n_random=1500):
    """A vocabulary in the style of a byte-level BPE: all single bytes, the fragments JSON text is
    made of (with and without leading blanks), and random printable / raw byte strings."""
    toks = [bytes([b]) for b in range(256)]
    frag = ['{"', '"}', '":', '": ', '",', '", "', '":"', "[]", "{}", "[[", "]]", "}}", "},", "],", ", ", " {", " [", "  ", "    ", "\n", "\n  ",
            "true", "false", "null", "tr", "ue", "nu", "ll", "fal", "se", '"name', "name", '"age"', "age", "tags", "kind", '"x"', '"x":', 'x":', "id",
            '"a"', '"bb"', "bb", '"fast"', "slow", "12", "30", "-1", ".5", "e3", "E-", "0.", "00", "1,", "1]", "1}", "1 ", "\\n", "\\u", "\\u00", "00e9",
            '\\"', "\\\\", "\\", ' "', '" ', "ok", "note", "pos", '"v":', "next", '"next":null}', "null}", '"mode":', "inner", '{"a":[1,2]}', '[1,2]',
            '":{"', "}]", "[{", '"k":{"a":[1,2]}', '", "b', " \t\r\n", "         ", "tags\":[\"a\",\"bb\"]"]
    toks += [f.encode() for f in frag]
    printable = np.frombuffer(bytes(range(0x20, 0x7F)), np.uint8)
    jsonish = np.frombuffer(b'{}[]:,"\\ 0123456789-.eEtruefalsn', np.uint8)
    for _ in range(n_random):
        ln = int(rng.integers(1, 9))
        kind = rng.random()
        src = jsonish if kind < 0.5 else printable if kind < 0.85 else np.arange(256, dtype=np.uint8)
        toks.append(bytes(src[rng.integers(0, len(src), ln)]))
    toks.append(b"")  # an empty piece is never allowed (tools/server_chat.h:556)
    off = np.zeros(len(toks) + 1, np.uint32)
    off[1:] = np.cumsum([len(t) for t in toks])
    return toks, off, np.frombuffer(b"".join(toks), np.uint8).copy()


@needs_ref
def test_table_mask_is_the_per_candidate_predicate():
    rng = np.random.default_rng(5)
    toks, off, by = json_vocab(rng)
    steps = 0
    for si, (schema, obj) in enumerate(SCHEMAS):
        jc = jcon.JsonConstraint(schema, obj, off, by)
        for doc in DOCS[si]:
            d = doc.encode()
            for cut in sorted(set(rng.integers(0, len(d) + 1, 14).tolist() + [0, len(d)])):
                text = d[:cut]
                table, dead, done, ts = jc.table(text)
                assert ts == ref_check(schema, obj, text) != F
                allowed, end = jcon.walk_mask(table, dead, off, by)
                for t, piece in enumerate(toks):
                    want = ref_check(schema, obj, text + piece) if piece else F
                    assert bool(allowed[t]) == (want != F), (si, text, piece, want)
                    if want != F:
                        assert bool(done[end[t]]) == (want == D), (si, text, piece, want)
                assert bool(done[0]) == (ts == D)
                steps += 1
        h, m = jc.cache_stats()
        assert h + m > 0
    assert steps > 200


def test_tables_are_cached_by_configuration():
    rng = np.random.default_rng(2)
    toks, off, by = json_vocab(rng, 200)
    jc = jcon.JsonConstraint("{}", True, off, by)
    a = jc.table('{"a": "hello')
    b = jc.table('{"a": "hello world, still inside the string')  # the same configuration
    assert np.array_equal(a[0], b[0]) and a[1] == b[1]
    assert jc.cache_stats() == (1, 1)
    with pytest.raises(ValueError):
        jc.table('{"a": 01')  # the text itself already fails


def test_schemas_without_a_finite_automaton_are_refused():
    for schema in ('{"anyOf":[{"type":"integer"},{"type":"number"}]}',
                   '{"oneOf":[{"type":"object","properties":{"a":{}}},{"type":"object","properties":{"b":{}}}]}',
                   '{"enum":[1,12]}'):
        with pytest.raises(jcon.Unsupported):
            jcon.JsonConstraint(schema, False, *EMPTY_VOCAB)
    jcon.JsonConstraint('{"enum":["1","12"]}', False, *EMPTY_VOCAB)  # (strings end with their quote)


def test_arguments_are_checked():
    lib = jcon._load()
    h = C.c_void_p()
    assert lib.arcs_jcon_create(None, 0, None, None, 0, C.byref(h)) == 1
    assert lib.arcs_jcon_check(None, b"", C.c_int64(0)) == -1
    bad = np.array([0, 3, 2], np.uint32)  # offsets that go backwards
    assert lib.arcs_jcon_create(b"{}", 0, bad.ctypes.data_as(C.c_void_p), np.zeros(4, np.uint8).ctypes.data_as(C.c_void_p), 2, C.byref(h)) == 1
    with pytest.raises(jcon.Unsupported, match="not JSON"):
        jcon.JsonConstraint("not json", False, *EMPTY_VOCAB)
    jc = jcon.JsonConstraint(json.dumps({}), False, *EMPTY_VOCAB)
    assert jc.check("[1]") == D


# ---- random schemas (the subset the checker knows) and documents that mostly fit them
def _rschema(rng, d=0):
    r=rng.random()
    if d>3 or r<0.25:
        t=rng.choice(["string","integer","number","boolean","null"])
        return {"type":str(t)}
    if r<0.35: return {}
    if r<0.45:
        opts=["a","bc","x y",1,25,None,True,-3.5]
        return {"enum":[opts[int(rng.integers(0,len(opts)))] for _ in range(int(rng.integers(1,4)))]}
    if r<0.5: return {"const": {"k":[1,"z"]}}
    if r<0.65:
        return {"type":"array","items":_rschema(rng, d+1),**({"minItems":int(rng.integers(0,3))} if rng.random()<0.5 else {}),**({"maxItems":int(rng.integers(1,4))} if rng.random()<0.5 else {})}
    if r<0.9:
        props={str(k):_rschema(rng, d+1) for k in rng.choice(["a","ab","b","name","n1"],int(rng.integers(0,4)),replace=False)}
        s={"type":"object","properties":props}
        if props and rng.random()<0.6: s["required"]=[str(k) for k in list(props)[:int(rng.integers(0,len(props)+1))]]
        c=rng.random()
        if c<0.3: s["additionalProperties"]=False
        elif c<0.5: s["additionalProperties"]=True
        elif c<0.7: s["additionalProperties"]=_rschema(rng, d+1)
        return s
    return {"anyOf":[_rschema(rng, d+1) for _ in range(int(rng.integers(1,4)))]}
def _rvalue(rng, s, d=0):
    # a value that often (not always) fits
    if "enum" in s: return s["enum"][int(rng.integers(0,len(s["enum"])))]
    if "const" in s: return s["const"]
    if "anyOf" in s: return _rvalue(rng, s["anyOf"][int(rng.integers(0,len(s["anyOf"])))],d+1)
    t=s.get("type")
    if t is None: t=str(rng.choice(["string","integer","object","array","null","boolean"]))
    if t=="string": return str(rng.choice(["","hi","a\"b","\\n x","ü"]))
    if t=="integer": return int(rng.integers(-50,500))
    if t=="number": return float(rng.choice([0.5,-12.25,3e5,7]))
    if t=="boolean": return bool(rng.integers(0,2))
    if t=="null": return None
    if t=="array": return [_rvalue(rng, s.get("items",{}),d+1) for _ in range(int(rng.integers(0,4)))] if d<4 else []
    if t=="object":
        o={}
        for k,v in s.get("properties",{}).items():
            if rng.random()<0.8: o[k]=_rvalue(rng, v,d+1)
        if rng.random()<0.3 and d<4: o["zz"]=_rvalue(rng, s["additionalProperties"] if isinstance(s.get("additionalProperties"),dict) else {},d+1)
        return o


@needs_ref
def test_random_schemas_against_the_reference_checker():
    rng = np.random.default_rng(123)
    pool = b'{}[]:,"\\ \n0123456789-+.eEtruefalsnabxyz'
    total = unsupported = 0
    for _ in range(160):
        s = _rschema(rng)
        sj = json.dumps(s)
        obj = bool(rng.integers(0, 2)) and s.get("type") == "object"
        try:
            jc = jcon.JsonConstraint(sj, obj, *EMPTY_VOCAB)
        except jcon.Unsupported:
            unsupported += 1
            continue
        for _rep in range(5):
            doc = json.dumps(_rvalue(rng, s), separators=(str(rng.choice([",", ", "])), str(rng.choice([":", ": "]))), ensure_ascii=False).encode()
            if rng.random() < 0.5 and len(doc):
                i = int(rng.integers(0, len(doc)))
                doc = doc[:i] + bytes([pool[int(rng.integers(0, len(pool)))]]) + doc[i + int(rng.integers(0, 2)):]
            for cut in range(len(doc) + 1):
                got, want = jc.check(doc[:cut]), ref_check(sj, obj, doc[:cut])
                assert got == want, (sj, obj, doc[:cut], got, want)
                total += 1
                if want == F:
                    break
    assert total > 4000 and unsupported < 40


@needs_ref
def test_random_schemas_table_masks_are_the_predicate():
    rng = np.random.default_rng(77)
    toks, off, by = json_vocab(rng, 500)
    total = 0
    for _ in range(60):
        s = _rschema(rng)
        sj = json.dumps(s)
        obj = bool(rng.integers(0, 2)) and s.get("type") == "object"
        try:
            jc = jcon.JsonConstraint(sj, obj, off, by)
        except jcon.Unsupported:
            continue
        doc = json.dumps(_rvalue(rng, s), separators=(str(rng.choice([",", ", "])), str(rng.choice([":", ": "]))), ensure_ascii=False).encode()
        if ref_check(sj, obj, doc) == F:
            continue
        for cut in sorted(set(rng.integers(0, len(doc) + 1, 3).tolist())):
            text = doc[:cut]
            if ref_check(sj, obj, text) == D:
                continue
            table, dead, done, _ts = jc.table(text)
            allowed, end = jcon.walk_mask(table, dead, off, by)
            for t, piece in enumerate(toks):
                want = ref_check(sj, obj, text + piece) if piece else F
                assert bool(allowed[t]) == (want != F), (sj, obj, text, piece, want)
                if want != F:
                    assert bool(done[end[t]]) == (want == D), (sj, obj, text, piece, want)
                total += 1
    assert total > 30000
