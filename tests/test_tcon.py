"""The Gemma tool-call form as a byte automaton (arcs_tcon_create + the arcs_jcon_* functions)
against the reference's tcon::GemmaCall::check (oracle/_ref, tools/tool_constraint.h:66-280): every
prefix of valid and damaged calls, and token by token over a synthetic vocabulary (the table's
mask bit must equal check(text + piece) != FAIL). No GPU needed."""
import json

import numpy as np
import pytest

import orc
from arcinfer_b200 import jcon
from test_jcon import damaged

F, P, D = jcon.FAIL, jcon.PARTIAL, jcon.DONE
Q = '<|"|>'
END = "<tool_call|>"

TOOLS = json.dumps([
    {"type": "function", "function": {"name": "get_weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}, "units": {"enum": ["c", "f", 3]},
                                         "opts": {"type": "object", "properties": {"deep": {"type": "boolean"}}, "additionalProperties": True}},
        "required": ["city"]}}},
    {"type": "function", "function": {"name": "get", "parameters": {"type": "object"}}},
    {"name": "edit.file", "parameters": {
        "$defs": {"R": {"type": "object", "properties": {"from": {"type": "integer"}, "to": {"type": "integer"}}, "required": ["from"]}},
        "type": "object", "properties": {"path": {"type": "string"}, "ranges": {"type": "array", "items": {"$ref": "#/$defs/R"}, "minItems": 1, "maxItems": 2},
                                         "mode": {"anyOf": [{"type": "null"}, {"const": "fast"}, {"type": "number"}]}},
        "required": ["path", "ranges"], "additionalProperties": False}},
    {"type": "function", "function": {"name": "noargs"}},
])  # fmt: skip

CALLS = [
    f"call:get_weather{{city:{Q}Oslo, NO{Q},days:3,units:{Q}c{Q}}}{END}",
    f"call:get_weather{{units:3,opts:{{deep:true,x-1:[1,-2.5,{Q}a<|b{Q},{{}}],y:null}},city:{Q}{Q}}}{END}",
    f"call:get{{anything:[{{k:{Q}v{Q}}},0,-0.5],$x:false}}{END}",
    f"call:get{{}}{END}",
    f"call:edit.file{{path:{Q}a/b.txt{Q},ranges:[{{from:1,to:2}},{{from:30}}],mode:{Q}fast{Q}}}{END}",
    f"call:edit.file{{ranges:[{{to:5,from:0}}],path:{Q}p{Q},mode:-1.25}}{END}",
    f"call:edit.file{{path:{Q}p{Q},ranges:[{{from:7}}],mode:null}}{END}",
    f"call:noargs{{free:1}}{END}",
]


def ref_check(text):
    return orc.ref.ref_tcon_check(0, TOOLS.encode(), text, len(text))


needs_ref = pytest.mark.skipif(orc.ref is None, reason="oracle/_ref/libarcs_ref.so not built (needs the reference tree)")
EMPTY_VOCAB = (np.zeros(1, np.uint32), np.zeros(0, np.uint8))


def test_calls_without_the_reference():
    tc = jcon.JsonConstraint.gemma_call(TOOLS, *EMPTY_VOCAB)
    for call in CALLS:
        assert tc.check(call) == D, call
        assert tc.check(call[:-1]) == P and tc.check(call + "x") == F
    for bad in ["call:nope{", "call:get_weather{}" + END, "call:get_weather{city:1", "call:get_weather{city:" + Q + "a" + Q + ",city:",
                "call:edit.file{path:" + Q + "p" + Q + ",ranges:[]", "call:get{a: 1", "call:get{a:1e", "call:get{:"]:
        assert tc.check(bad) == F, bad
    with pytest.raises(jcon.Unsupported):
        jcon.JsonConstraint.gemma_call(json.dumps([{"name": "t", "parameters": {"type": "object", "properties": {"v": {"anyOf": [{"type": "integer"}, {"type": "number"}]}}}}]), *EMPTY_VOCAB)
    lib = jcon._load()
    import ctypes as C

    h = C.c_void_p()
    assert lib.arcs_tcon_create(7, b"[]", None, None, 0, C.byref(h)) == 1  # no such form


@needs_ref
def test_every_prefix_against_the_reference_checker():
    rng = np.random.default_rng(21)
    tc = jcon.JsonConstraint.gemma_call(TOOLS, *EMPTY_VOCAB)
    n = 0
    for call in CALLS:
        for text in [call.encode()] + damaged(call, rng, 60):
            for cut in range(len(text) + 1):
                got, want = tc.check(text[:cut]), ref_check(text[:cut])
                assert got == want, (text[:cut], got, want)
                n += 1
                if want == F:
                    break
            if cut < len(text):
                assert tc.check(text) == ref_check(text) == F
    assert n > 5000


def call_vocab(rng, n_random=1200):
    toks = [bytes([b]) for b in range(256)]
    frag = ["call:", "call:get", "get_", "weather", "_weather{", "edit", ".file", "edit.file{", "noargs", "{}", "}" + END, END, "<tool", "_call|>", "<|", '"|>', Q, Q + ",", "," , ":" + Q,
            "city", "city:", "days:", "days:3", "units", "opts:{", "deep:", "true", "false", "null", "tru", "path:", "ranges:[", "ranges:[{", "from:", "to:", "{from:", "mode:", "mode:" + Q + "fast" + Q,
            "fast", "}]", "},{", "]}", "}}", "[1,", "-2.5", "0.", "12", "3}", "3,", ":[", "x-1:", "$x:", "a<|b", "<", "|", "free:1"]
    toks += [f.encode() for f in frag]
    src = np.frombuffer(b'call:get_wathrdi.fnos{}[],<|">-0123456789$xyzk', np.uint8)
    printable = np.frombuffer(bytes(range(0x20, 0x7F)), np.uint8)
    for _ in range(n_random):
        ln = int(rng.integers(1, 8))
        a = src if rng.random() < 0.7 else printable
        toks.append(bytes(a[rng.integers(0, len(a), ln)]))
    toks.append(b"")
    off = np.zeros(len(toks) + 1, np.uint32)
    off[1:] = np.cumsum([len(t) for t in toks])
    return toks, off, np.frombuffer(b"".join(toks), np.uint8).copy()


@needs_ref
def test_table_mask_is_the_per_candidate_predicate():
    rng = np.random.default_rng(8)
    toks, off, by = call_vocab(rng)
    tc = jcon.JsonConstraint.gemma_call(TOOLS, off, by)
    steps = 0
    for call in CALLS:
        d = call.encode()
        for cut in sorted(set(rng.integers(0, len(d), 16).tolist() + [0, len(d) - 1])):
            text = d[:cut]
            table, dead, done, ts = tc.table(text)
            assert ts == ref_check(text) == P
            allowed, end = jcon.walk_mask(table, dead, off, by)
            for t, piece in enumerate(toks):
                want = ref_check(text + piece) if piece else F
                assert bool(allowed[t]) == (want != F), (text, piece, want)
                if want != F:
                    assert bool(done[end[t]]) == (want == D), (text, piece, want)
            steps += 1
    assert steps > 60


# ---------------------------------------------------------------- the Qwen 3.x form (tools/tool_constraint.h:285-371)
QTOOLS = json.dumps([
    {"type": "function", "function": {"name": "search", "parameters": {
        "type": "object", "properties": {"query": {"type": "string"}, "limit": {"type": "integer"}, "exact": {"type": "boolean"},
                                         "filters": {"type": "object", "properties": {"lang": {"enum": ["en", "de"]}}, "required": ["lang"]},
                                         "tags": {"type": "array", "items": {"type": "string"}, "maxItems": 3}, "free": {}},
        "required": ["query"]}}},
    {"type": "function", "function": {"name": "search_all", "parameters": {"type": "object", "additionalProperties": {"type": "number"}}}},
    {"name": "ping"},
])  # fmt: skip

# (a number at the very end of a value is still PARTIAL for jcon::Checker - more digits could follow - so the
#  reference takes a numeric parameter only with a blank behind it, besides the one newline it strips: :364-368)
QCALLS = [
    "\n<function=search>\n<parameter=query>\nhello <b>world</b> 1 < 2\n</parameter>\n<parameter=limit>\n10\n\n</parameter>\n</function>\n</tool_call>",
    "<function=search><parameter=exact>true</parameter><parameter=query>q</parameter> <parameter=filters>{\"lang\": \"de\"}\n</parameter></function></tool_call>",
    "<function=search>\n<parameter=tags>\n[\"a<\", \"</param\", \"x\"]\n</parameter>\n<parameter=query>\n\n</parameter>\n<parameter=free>\nany {text} here</parameter>\n</function>\n</tool_call>",
    " <function=search_all>\n<parameter=a>\n-1.5e3 \n</parameter>\n<parameter=b>2 </parameter>\n</function> </tool_call>",
    "<function=ping>\n</function>\n</tool_call>",
    "<function=search>\n<parameter=limit>\n 7\n\n</parameter>\n<parameter=query>\nx</parameter>\n</function>\n</tool_call>",
]


def ref_qcheck(text):
    return orc.ref.ref_tcon_check(1, QTOOLS.encode(), text, len(text))


def test_qwen_calls_without_the_reference():
    tc = jcon.JsonConstraint.qwen_call(QTOOLS, *EMPTY_VOCAB)
    for call in QCALLS:
        assert tc.check(call) == D, call
        assert tc.check(call[:-1]) == P and tc.check(call + "x") == F
    for bad in ["<function=nope", "<function=search>\n</function>", "<function=search>\n<parameter=limit>\n1.5\n</parameter>",
                "<function=search>\n<parameter=query>a<parameter=", "<function=search>\n<parameter=limit>1</parameter><parameter=limit>",
                "   <function=", "<function=search>\n\n\n<", "<function=ping></function></tool_call> \n\n",
                "<function=search>\n<parameter=limit>\n10\n</parameter>"]:
        assert tc.check(bad) == F, bad


@needs_ref
def test_qwen_every_prefix_against_the_reference_checker():
    rng = np.random.default_rng(33)
    tc = jcon.JsonConstraint.qwen_call(QTOOLS, *EMPTY_VOCAB)
    n = 0
    for call in QCALLS:
        for text in [call.encode()] + damaged(call, rng, 80):
            for cut in range(len(text) + 1):
                got, want = tc.check(text[:cut]), ref_qcheck(text[:cut])
                assert got == want, (text[:cut], got, want)
                n += 1
                if want == F:
                    break
            if cut < len(text):
                assert tc.check(text) == ref_qcheck(text) == F
    assert n > 8000


def qwen_vocab(rng, n_random=1200):
    toks = [bytes([b]) for b in range(256)]
    frag = ["<function=", "<function=search", "search", "_all", ">\n", "<parameter=", "<parameter=query>", "query", "limit", ">\n10\n", "</parameter>", "</parameter>\n", "\n</parameter>",
            "</", "</param", "eter>", "<param", "</function>", "</function>\n", "</tool_call>", "\n</tool_call>", "<", ">", "\n", "\n\n", " ", "  ", "true", "false", "tru", "10", "-1", ".5e3",
            '{"lang"', '": "de"}', '["a<"', ', "', '"]', "hello", " world", "<b>", "exact", "filters", "tags", "free", "ping", "a>", "b>2", "e3 \n"]
    toks += [f.encode() for f in frag]
    src = np.frombuffer(b'<>/=\n function parameter search query limit 0123456789-.e"{}[],:truefals', np.uint8)
    printable = np.frombuffer(bytes(range(0x20, 0x7F)), np.uint8)
    for _ in range(n_random):
        ln = int(rng.integers(1, 8))
        a = src if rng.random() < 0.7 else printable
        toks.append(bytes(a[rng.integers(0, len(a), ln)]))
    toks.append(b"")
    off = np.zeros(len(toks) + 1, np.uint32)
    off[1:] = np.cumsum([len(t) for t in toks])
    return toks, off, np.frombuffer(b"".join(toks), np.uint8).copy()


@needs_ref
def test_qwen_table_mask_is_the_per_candidate_predicate():
    rng = np.random.default_rng(9)
    toks, off, by = qwen_vocab(rng)
    tc = jcon.JsonConstraint.qwen_call(QTOOLS, off, by)
    steps = 0
    for call in QCALLS:
        d = call.encode()
        for cut in sorted(set(rng.integers(0, len(d), 18).tolist() + [0, len(d) - 1])):
            text = d[:cut]
            table, dead, done, ts = tc.table(text)
            assert ts == ref_qcheck(text) == P
            allowed, end = jcon.walk_mask(table, dead, off, by)
            for t, piece in enumerate(toks):
                want = ref_qcheck(text + piece) if piece else F
                assert bool(allowed[t]) == (want != F), (text, piece, want)
                if want != F:
                    assert bool(done[end[t]]) == (want == D), (text, piece, want)
            steps += 1
    assert steps > 60


# ---- random parameter schemas: calls written in either form, damaged, every prefix
def _gemma_text(v):
    if isinstance(v, str):
        return Q + v + Q
    if isinstance(v, bool):
        return "true" if v else "false"
    if v is None:
        return "null"
    if isinstance(v, (int, float)):
        s = repr(v)
        return s if "e" not in s and "E" not in s else str(int(v))
    if isinstance(v, list):
        return "[" + ",".join(_gemma_text(x) for x in v) + "]"
    return "{" + ",".join(k + ":" + _gemma_text(x) for k, x in v.items()) + "}"


def _qwen_text(name, params, args):
    out = "<function=" + name + ">\n"
    for k, v in args.items():
        addl = params.get("additionalProperties")
        vs = params.get("properties", {}).get(k, addl if isinstance(addl, dict) else {})
        raw = vs.get("type") == "string" or "type" not in vs
        body = (v if isinstance(v, str) else json.dumps(v)) if raw else json.dumps(v) + " "
        out += "<parameter=" + k + ">\n" + body + "\n</parameter>\n"
    return out + "</function>\n</tool_call>"


@needs_ref
@pytest.mark.parametrize("kind", [0, 1])
def test_random_parameter_schemas_against_the_reference_checker(kind):
    from test_jcon import _rschema, _rvalue

    rng = np.random.default_rng(5 + kind)
    pool = b'{}[]:,<|">/=\n 0123456789-.truefalsnabxyz'
    total = done = 0
    for _ in range(90):
        params = _rschema(rng, 1)
        while params.get("type") != "object":
            params = _rschema(rng, 1)
        tools = json.dumps([{"type": "function", "function": {"name": "tool_a", "parameters": params}}, {"name": "tool", "parameters": {"type": "object"}}])
        try:
            tc = (jcon.JsonConstraint.gemma_call if kind == 0 else jcon.JsonConstraint.qwen_call)(tools, *EMPTY_VOCAB)
        except jcon.Unsupported:
            continue
        for _rep in range(4):
            args = _rvalue(rng, params)
            doc = (("call:tool_a" + _gemma_text(args) + END) if kind == 0 else _qwen_text("tool_a", params, args)).encode()
            if rng.random() < 0.5:
                i = int(rng.integers(0, len(doc)))
                doc = doc[:i] + bytes([pool[int(rng.integers(0, len(pool)))]]) + doc[i + int(rng.integers(0, 2)):]
            for cut in range(len(doc) + 1):
                got, want = tc.check(doc[:cut]), orc.ref.ref_tcon_check(kind, tools.encode(), doc[:cut], cut)
                assert got == want, (kind, tools, doc[:cut], got, want)
                total += 1
                done += want == D
                if want == F:
                    break
    assert total > 5000 and done > 20
