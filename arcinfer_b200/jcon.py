"""Constrained JSON output: the binding of arcs_jcon_* (include/arcsample.h). Host work only;
numpy in, numpy out. `JsonConstraint.table(text)` gives what `arcs_dfa_mask` needs for the step
after `text`; `check(text)` is jcon::Checker::check of tools/json_constraint.h:37-47."""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libarcsample.so")

FAIL, PARTIAL, DONE = 0, 1, 2
ERR_UNSUPPORTED = 8

_lib = None


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `make -C arcinfer_b200/csrc`; there is no fallback")
        _lib = C.CDLL(LIB_PATH)
        _lib.arcs_jcon_why.restype = C.c_char_p
        _lib.arcs_jcon_destroy.restype = None
        _lib.arcs_jcon_cache_stats.restype = None
    return _lib


class Unsupported(ValueError):
    """The schema (or one step's table) is outside what the automaton expresses: keep the
    per-candidate predicate in ranked order for it."""


class JsonConstraint:
    def __init__(self, schema_json, object_only, byte_off, bytes_):
        """schema_json: the schema's JSON text; object_only: json_object mode
        (tools/server_chat.h:30-31). byte_off uint32 [V+1], bytes_ uint8: the vocabulary."""
        lib = _load()
        self._h = C.c_void_p()
        byte_off = np.ascontiguousarray(byte_off, dtype=np.uint32)
        bytes_ = np.ascontiguousarray(bytes_, dtype=np.uint8)
        self.V = len(byte_off) - 1
        rc = lib.arcs_jcon_create(schema_json.encode(), int(bool(object_only)), byte_off.ctypes.data_as(C.c_void_p),
                                  bytes_.ctypes.data_as(C.c_void_p), self.V, C.byref(self._h))
        if rc == ERR_UNSUPPORTED:
            why = lib.arcs_jcon_why(self._h).decode()
            self.close()
            raise Unsupported(why)
        if rc != 0:
            raise ValueError(f"arcs_jcon_create failed with code {rc}")

    @classmethod
    def qwen_call(cls, tools_json, byte_off, bytes_):
        """The Qwen 3.x tool-call form (tcon::QwenCall, tools/tool_constraint.h:285-371): texts are
        what follows <tool_call>."""
        return cls.gemma_call(tools_json, byte_off, bytes_, kind=1)

    @classmethod
    def gemma_call(cls, tools_json, byte_off, bytes_, kind=0):
        """The Gemma tool-call form (tcon::GemmaCall, tools/tool_constraint.h:66-280): texts are
        what follows <|tool_call>; tools_json: the request's "tools" array as JSON text."""
        lib = _load()
        self = cls.__new__(cls)
        self._h = C.c_void_p()
        byte_off = np.ascontiguousarray(byte_off, dtype=np.uint32)
        bytes_ = np.ascontiguousarray(bytes_, dtype=np.uint8)
        self.V = len(byte_off) - 1
        rc = lib.arcs_tcon_create(kind, tools_json.encode(), byte_off.ctypes.data_as(C.c_void_p), bytes_.ctypes.data_as(C.c_void_p), self.V, C.byref(self._h))
        if rc == ERR_UNSUPPORTED:
            why = lib.arcs_jcon_why(self._h).decode()
            self.close()
            raise Unsupported(why)
        if rc != 0:
            raise ValueError(f"arcs_tcon_create failed with code {rc}")
        return self

    def close(self):
        if getattr(self, "_h", None):
            _load().arcs_jcon_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        self.close()

    def check(self, text):
        b = text if isinstance(text, bytes) else text.encode()
        return _load().arcs_jcon_check(self._h, b, C.c_int64(len(b)))

    def table(self, text):
        """(table uint16 [S,256], dead, done uint8 [S], check(text)) for the step after `text`;
        state 0 is the start. The arrays are copies."""
        b = text if isinstance(text, bytes) else text.encode()
        tp, dn = C.POINTER(C.c_uint16)(), C.POINTER(C.c_uint8)()
        S, dead, ts = C.c_int32(), C.c_int32(), C.c_int32()
        rc = _load().arcs_jcon_table(self._h, b, C.c_int64(len(b)), C.byref(tp), C.byref(S), C.byref(dead), C.byref(dn), C.byref(ts))
        if rc == ERR_UNSUPPORTED:
            raise Unsupported("this step needs more states than a table holds")
        if rc != 0:
            raise ValueError(f"arcs_jcon_table failed with code {rc} (check(text) = {ts.value})")
        table = np.ctypeslib.as_array(tp, shape=(S.value, 256)).copy()
        done = np.ctypeslib.as_array(dn, shape=(S.value,)).copy()
        return table, dead.value, done, ts.value

    def cache_stats(self):
        h, m = C.c_int64(), C.c_int64()
        _load().arcs_jcon_cache_stats(self._h, C.byref(h), C.byref(m))
        return h.value, m.value


def walk_mask(table, dead, byte_off, bytes_):
    """The mask arcs_dfa_mask computes, on the host with numpy (for tests and small vocabularies):
    bool [V], token t allowed iff it is not empty and its bytes never lead to `dead` from state 0."""
    V = len(byte_off) - 1
    lens = np.diff(byte_off.astype(np.int64))
    st = np.zeros(V, dtype=np.int64)
    for d in range(int(lens.max()) if V else 0):
        live = (lens > d) & (st != dead)
        idx = np.nonzero(live)[0]
        st[idx] = table[st[idx], bytes_[byte_off[idx].astype(np.int64) + d]]
    return (lens > 0) & (st != dead), st
