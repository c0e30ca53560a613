// Byte-level automaton for constrained JSON output: the prefix checker of the reference
// (jcon::Checker::check, tools/json_constraint.h:37-281) restated as an INCREMENTAL pushdown
// machine, so that "is text + piece still a prefix of a matching document" can be answered for a
// whole vocabulary at once: from the configuration after the current answer text, the byte
// transitions reachable within one token are expanded into the [S][256] table that arcs_dfa_mask
// walks on the GPU (mask bit t == (check(text + piece(t)) != FAIL), tools/server_chat.h:553-557).
//
// The reference re-parses the whole answer for every candidate token; here the answer is fed once,
// byte by byte, and a configuration (a stack of frames: where in which schema node the text
// stands) is all that the future depends on. Equal configurations are one automaton state.
//
// What is reproduced, rule for rule (line numbers of tools/json_constraint.h): unbounded leading
// whitespace, at most 2 trailing (:37-47); at most 8 whitespace characters in a row inside
// objects and arrays (:66-70); nesting deeper than 32 fails (:93); $ref one level deep (:53-64);
// anyOf / oneOf (:96-108); enum / const against the compact JSON text of the options (:112-124);
// type dispatch on the first character, integer without '.' / 'e' (:125-168); strings with their
// escapes, control characters refused (:170-198); objects with properties / required /
// additionalProperties, used keys, comma only where a key can follow (:199-255); arrays with
// items / minItems / maxItems (:256-281).
//
// Two constructions of the reference have no finite-lookahead automaton and are refused at
// construction (supported() == false; the caller then keeps calling its predicate per candidate,
// in ranked order): anyOf / oneOf whose branches can start with the same character (the reference
// tries them in order and lets the first that completes win, whatever follows), and an enum in
// which one option's text is a proper prefix of another's (possible for numbers only).
#pragma once
#include <algorithm>
#include <cstring>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "mini_json.hpp"

namespace arcinfer_b200 {
namespace jcon {

enum Res { FAIL = 0, PARTIAL = 1, DONE = 2 };  // jcon::Res of the reference

struct Frame {
  uint8_t type = 0;   // FrameType
  uint8_t sub = 0;    // phase / state inside the frame
  uint8_t ws = 0;     // whitespace characters of the current gap
  uint8_t flag = 0;   // NUM: integer only; STR: an object key; OBJ: a key the schema does not name was closed during a table walk
  int32_t node = -1;  // schema node (index into Automaton::nodes_), -1: the "any value" schema
  int32_t n = 0;      // ARR: elements so far (capped where more make no difference); LIT: position; STR: hex digits left
  int32_t depth = 0;  // OBJ / ARR: nesting depth of this value
  std::string text;   // STR (key): decoded key so far; ENUM: text consumed; LIT: the literal
  std::vector<std::string> seen;  // OBJ: keys used, sorted
};
using Config = std::vector<Frame>;

enum FrameType : uint8_t { F_TOP = 1, F_NUM, F_STR, F_LIT, F_ENUM, F_OBJ, F_ARR, F_GSTR, F_GOBJ };
// F_TOP.sub (G_*: the Gemma tool-call form)
enum : uint8_t { T_LEAD = 0, T_VALUE = 1, T_TRAIL = 2, G_CALL = 3, G_NAME = 4, G_CLOSE = 5, G_END = 6 };
// F_GSTR.sub: inside the opening <|"|>, inside the text (n: how much of the closing <|"|> has been seen)
enum : uint8_t { GS_OPEN = 0, GS_BODY = 1 };
// F_GOBJ.sub
enum : uint8_t { GO_OPEN = 0, GO_KEY, GO_AFTER_COLON, GO_IN_VALUE, GO_AFTER_VALUE };
// F_NUM.sub
enum : uint8_t { N_MINUS = 0, N_ZERO, N_INT, N_DOT, N_FRAC, N_E, N_ESIGN, N_EXP };
// F_STR.sub
enum : uint8_t { S_NORMAL = 0, S_ESC, S_HEX };
// F_OBJ.sub
enum : uint8_t { O_OPEN = 0, O_AFTER_COMMA, O_IN_KEY, O_AFTER_KEY, O_AFTER_COLON, O_IN_VALUE, O_AFTER_VALUE };
// F_ARR.sub
enum : uint8_t { A_OPEN = 0, A_IN_VALUE, A_AFTER_ELEM, A_AFTER_COMMA };

constexpr const char* kGemmaQuote = "<|\"|>";       // tcon::GemmaCall::kQ
constexpr const char* kGemmaClose = "<tool_call|>";  // tcon::GemmaCall::kClose
constexpr const char* kOtherKey = "\x01other";  // a key no property and no used key starts with (table walks only)

inline bool is_ws(uint8_t c) { return c == ' ' || c == '\n' || c == '\r' || c == '\t'; }


class Automaton {
 public:
  using State = Config;
  enum Dialect { JSON = 0, GEMMA = 1 };
  // schema_json: the JSON schema as text ("{}" = any value); object_only: the value must be an
  // object (json_object mode), as jcon::Checker(schema, object_only)
  Automaton(const std::string& schema_json, bool object_only) : object_only_(object_only) {
    if (!JVal::parse(schema_json, root_)) {
      why_ = "the schema is not JSON";
      return;
    }
    std::vector<const JVal*> path;
    supported_ = vet(root_, path, root_);
  }
  // The Gemma 4 tool-call form (tcon::GemmaCall, tools/tool_constraint.h:66-280): the text after
  // <|tool_call> is call:NAME{key:value,...}<tool_call|>, keys bare words, strings between
  // <|"|> delimiters, no whitespace; tools_json: the request's "tools" (:45-51).
  Automaton(const std::string& tools_json, Dialect gemma) : dialect_(gemma) {
    if (!JVal::parse(tools_json, root_)) {
      why_ = "the tool list is not JSON";
      return;
    }
    supported_ = true;
    for (const JVal& t : root_.a) {
      const JVal& f = t.has("function") ? t["function"] : t;
      if (f["name"].str().empty()) continue;
      const JVal* params = f["parameters"].is_object() ? &f["parameters"] : &any_schema();
      tools_.push_back({f["name"].str(), params});
      std::vector<const JVal*> path;
      supported_ = supported_ && vet(*params, path, *params);
    }
  }
  bool supported() const { return supported_; }
  const std::string& why_not() const { return why_; }

  Config start() const {
    Config c(1);
    c[0].type = F_TOP;
    c[0].sub = dialect_ == GEMMA ? G_CALL : T_LEAD;
    return c;
  }
  // one more byte of the answer; false: no continuation fits (FAIL). `walk`: the call is part of a
  // table expansion, where keys that no property and no used key starts with are folded into one.
  bool step(Config& st, uint8_t c, bool walk = false) const;
  // PARTIAL or DONE for a configuration that has not failed (tools/json_constraint.h:37-47)
  Res classify(const Config& st) const { return st.size() == 1 && st[0].sub == (dialect_ == GEMMA ? G_END : T_TRAIL) ? DONE : PARTIAL; }
  // Checker::check: FAIL / PARTIAL / DONE for a whole text
  Res check(const std::string& text) const {
    Config st = start();
    for (unsigned char ch : text)
      if (!step(st, ch)) return FAIL;
    return classify(st);
  }

  // The transition table for one decoding step, expanded on demand: only the transitions some
  // token of the vocabulary takes from `from` (the configuration after the answer so far) are
  // worked out, by one walk over the vocabulary in byte order (tokens that share a prefix share
  // the steps over it); every other entry of the table leads to `dead`, which no token reaches
  // by it. table: [n_states][256] next states, row `dead` maps to itself; state 0 is `from`.
  // done[s]: the answer is complete in state s (the server then ends it,
  // tools/server_chat.h:550-551). Returns false when more than max_states states are met (the
  // caller keeps its per-candidate predicate for this step).
  struct Table {
    std::vector<uint16_t> next;  // [n_states][256]
    std::vector<uint8_t> done;   // [n_states]
    int n_states = 0, dead = 0, start = 0;
  };
  // a vocabulary in byte order (built once): token t is bytes[byte_off[t] .. byte_off[t + 1])
  struct Vocab {
    const uint32_t* byte_off = nullptr;
    const uint8_t* bytes = nullptr;
    std::vector<int32_t> order;  // token ids sorted by their byte strings
    Vocab(const uint32_t* off, const uint8_t* by, int32_t V) : byte_off(off), bytes(by), order((size_t)V) {
      for (int32_t t = 0; t < V; ++t) order[(size_t)t] = t;
      std::sort(order.begin(), order.end(), [&](int32_t x, int32_t y) {
        const uint32_t lx = off[x + 1] - off[x], ly = off[y + 1] - off[y];
        const int c = std::memcmp(by + off[x], by + off[y], std::min(lx, ly));
        return c < 0 || (c == 0 && lx < ly);
      });
    }
  };
  bool table(const Config& from, const Vocab& vocab, Table& out, int max_states = 8192) const;
  std::string key(const Config& st) const;
  // whether an object of this schema takes keys it does not name (tools/json_constraint.h:204)
  static bool any_key_of_public(const JVal& sc) { return any_key_of(sc); }

 private:
  JVal root_;
  Dialect dialect_ = JSON;
  bool object_only_ = false, supported_ = false;
  std::string why_;
  std::vector<std::pair<std::string, const JVal*>> tools_;  // (GEMMA) name, parameters
  // the schema `$ref`s are resolved against: the schema itself, or the parameters of the tool the call names
  const JVal& root_of(const Config& st) const { return dialect_ == GEMMA && st[0].node >= 0 ? node(st[0].node) : root_; }
  mutable std::vector<const JVal*> nodes_;

  int node_id(const JVal* p) const {
    for (size_t i = 0; i < nodes_.size(); ++i)
      if (nodes_[i] == p) return (int)i;
    nodes_.push_back(p);
    return (int)nodes_.size() - 1;
  }
  static const JVal& any_schema() {
    static const JVal any = [] {
      JVal v;
      v.t = JVal::Object;
      return v;
    }();
    return any;
  }
  const JVal& node(int id) const { return id < 0 ? any_schema() : *nodes_[(size_t)id]; }
  // :53-64, one level
  static const JVal& resolve(const JVal& sc, const JVal& root) {
    const std::string ref = sc["$ref"].str();
    if (ref.empty()) return sc;
    for (const char* pre : {"#/$defs/", "#/definitions/"}) {
      const std::string p = pre;
      if (ref.compare(0, p.size(), p) == 0) return root[p.substr(2, p.size() - 3)][ref.substr(p.size())];
    }
    return root;
  }
  static bool has_type(const JVal& sc, const char* t) {  // :71-80
    const JVal& ty = sc["type"];
    const bool num = std::strcmp(t, "number") == 0;
    if (ty.is_string()) return ty.s == t || (num && ty.s == "integer");
    if (ty.is_array()) {
      for (const JVal& x : ty.a)
        if (x.str() == t || (num && x.str() == "integer")) return true;
      return false;
    }
    return true;
  }
  static bool integer_only(const JVal& sc) {  // :81-90
    const JVal& ty = sc["type"];
    if (ty.is_string()) return ty.s == "integer";
    if (ty.is_array()) {
      bool num = false, integer = false;
      for (const JVal& x : ty.a) {
        num = num || x.str() == "number";
        integer = integer || x.str() == "integer";
      }
      return integer && !num;
    }
    return false;
  }
  static const JVal* alternatives(const JVal& sc) {  // :96-97: anyOf before oneOf
    for (const char* k : {"anyOf", "oneOf"})
      if (sc[k].is_array()) return &sc[k];
    return nullptr;
  }
  static bool is_enum(const JVal& sc) { return sc["enum"].is_array() || sc.has("const"); }
  // the text an allowed value is written as: compact JSON (:113-115), or, in the Gemma form, a
  // string between its delimiters and anything else as JSON (tools/tool_constraint.h:171-174)
  std::string text_of(const JVal& v) const {
    if (dialect_ == GEMMA && v.is_string()) return std::string(kGemmaQuote) + v.s + kGemmaQuote;
    return v.dump();
  }
  std::vector<std::string> options(const JVal& sc) const {
    std::vector<std::string> o;
    if (sc.has("const")) o.push_back(text_of(sc["const"]));
    for (const JVal& e : sc["enum"].a) o.push_back(text_of(e));
    return o;
  }
  struct CharSet {
    uint64_t w[4] = {0, 0, 0, 0};
    void add(unsigned c) { w[c >> 6] |= 1ull << (c & 63); }
    bool has(unsigned c) const { return (w[c >> 6] >> (c & 63)) & 1ull; }
    void all() { w[0] = w[1] = w[2] = w[3] = ~0ull; }
    void join(const CharSet& o) {
      for (int i = 0; i < 4; ++i) w[i] |= o.w[i];
    }
    bool meets(const CharSet& o) const { return (w[0] & o.w[0]) | (w[1] & o.w[1]) | (w[2] & o.w[2]) | (w[3] & o.w[3]); }
  };
  // the characters a value of this schema can start with (a superset: a cycle of references gives all)
  CharSet first_chars(const JVal& sc0, std::vector<const JVal*>& path, const JVal& root) const {
    CharSet cs;
    const JVal& sc = resolve(sc0, root);
    if (std::find(path.begin(), path.end(), &sc) != path.end() || path.size() > 64) {
      cs.all();
      return cs;
    }
    path.push_back(&sc);
    if (const JVal* alt = alternatives(sc)) {
      for (const JVal& br : alt->a) cs.join(first_chars(br, path, root));
    } else if (is_enum(sc)) {
      for (const std::string& o : options(sc))
        if (!o.empty()) cs.add((unsigned char)o[0]);
    } else {
      if (has_type(sc, "object")) cs.add('{');
      if (has_type(sc, "array")) cs.add('[');
      if (has_type(sc, "string")) cs.add(dialect_ == GEMMA ? '<' : '"');
      if (has_type(sc, "number")) {
        cs.add('-');
        for (char d = '0'; d <= '9'; ++d) cs.add((unsigned char)d);
      }
      if (has_type(sc, "boolean")) {
        cs.add('t');
        cs.add('f');
      }
      if (has_type(sc, "null")) cs.add('n');
    }
    path.pop_back();
    return cs;
  }
  // every schema node a value can be checked against: are its alternatives told apart by their
  // first character, and is no enum option a proper prefix of another?
  bool vet(const JVal& sc0, std::vector<const JVal*>& path, const JVal& root) {
    const JVal& sc = resolve(sc0, root);
    if (std::find(path.begin(), path.end(), &sc) != path.end()) return true;
    if (path.size() > 256) {
      why_ = "schema nested too deep";
      return false;
    }
    path.push_back(&sc);
    bool ok = true;
    if (const JVal* alt = alternatives(sc)) {
      std::vector<CharSet> sets;
      for (const JVal& br : alt->a) {
        std::vector<const JVal*> p2;
        sets.push_back(first_chars(br, p2, root));
      }
      for (size_t i = 0; i < sets.size() && ok; ++i)
        for (size_t j = i + 1; j < sets.size() && ok; ++j)
          if (sets[i].meets(sets[j])) {
            ok = false;
            why_ = "anyOf / oneOf branches that can start with the same character";
          }
      for (const JVal& br : alt->a) ok = ok && vet(br, path, root);
    } else if (is_enum(sc)) {
      const std::vector<std::string> o = options(sc);
      for (size_t i = 0; i < o.size() && ok; ++i)
        for (size_t j = 0; j < o.size() && ok; ++j)
          if (i != j && o[i].size() < o[j].size() && o[j].compare(0, o[i].size(), o[i]) == 0) {
            ok = false;
            why_ = "an enum option that is a proper prefix of another";
          }
    } else {
      for (const auto& kv : sc["properties"].o) ok = ok && vet(kv.second, path, root);
      if (sc["additionalProperties"].is_object()) ok = ok && vet(sc["additionalProperties"], path, root);
      if (sc["items"].is_object()) ok = ok && vet(sc["items"], path, root);
    }
    path.pop_back();
    return ok;
  }

  // ---- stepping (json_automaton_step.hpp)
  bool start_value(Config& st, int node, int depth, uint8_t c) const;
  bool complete(Config& st, bool walk) const;
  static bool any_key_of(const JVal& sc) {  // :204
    const JVal& props = sc["properties"];
    const JVal& addl = sc["additionalProperties"];
    return addl.is_object() || addl.as_bool(false) || (!props.is_object() && !addl.is_bool());
  }
  bool key_allowed(const Frame& obj, const std::string& k, bool prefix) const;
  bool step_gemma_top(Config& st, uint8_t c) const;
  bool step_gemma_object(Config& st, uint8_t c, bool walk) const;
};

// a configuration as a string: equal strings, equal futures
inline std::string config_key(const Config& st);
inline std::string Automaton::key(const Config& st) const { return config_key(st); }
inline std::string config_key(const Config& st) {
  std::string k;
  for (const Frame& f : st) {
    k.push_back((char)f.type);
    k.push_back((char)f.sub);
    k.push_back((char)f.ws);
    k.push_back((char)f.flag);
    k.append(reinterpret_cast<const char*>(&f.node), 4);
    k.append(reinterpret_cast<const char*>(&f.n), 4);
    k.append(reinterpret_cast<const char*>(&f.depth), 4);
    const uint32_t tl = (uint32_t)f.text.size(), ns = (uint32_t)f.seen.size();
    k.append(reinterpret_cast<const char*>(&tl), 4);
    k += f.text;
    k.append(reinterpret_cast<const char*>(&ns), 4);
    for (const std::string& x : f.seen) {
      const uint32_t xl = (uint32_t)x.size();
      k.append(reinterpret_cast<const char*>(&xl), 4);
      k += x;
    }
  }
  return k;
}

// The expansion itself, for any machine M with a state type, `bool step(State&, uint8_t, bool walk)`,
// `std::string key(const State&)` (equal keys, equal futures) and `Res classify(const State&)`.
template <class M>
bool build_table(const M& m, const typename M::State& from, const Automaton::Vocab& vocab, Automaton::Table& out, int max_states) {
  using State = typename M::State;
  if (max_states > 65534) max_states = 65534;
  std::unordered_map<std::string, int> ids;
  std::vector<State> cfg;
  std::vector<std::vector<int>> next;  // [state][256]: -2 not worked out, -1 dead
  ids.emplace(m.key(from), 0);
  cfg.push_back(from);
  next.emplace_back(256, -2);
  bool full = false;
  auto trans = [&](int s, uint8_t c) -> int {
    int& slot = next[(size_t)s][c];
    if (slot != -2) return slot;
    State t = cfg[(size_t)s];
    if (!m.step(t, c, true)) return slot = -1;
    const std::string key = m.key(t);
    auto it = ids.find(key);
    if (it == ids.end()) {
      if ((int)cfg.size() >= max_states) {
        full = true;
        return -1;
      }
      it = ids.emplace(key, (int)cfg.size()).first;
      cfg.push_back(std::move(t));
      next.emplace_back(256, -2);
    }
    return next[(size_t)s][c] = it->second;  // (`slot` may dangle after the push above)
  };
  // tokens order[lo, hi) share their first `depth` bytes, which lead from `from` to `state`
  struct Span {
    size_t lo, hi;
    uint32_t depth;
    int state;
  };
  std::vector<Span> todo{{0, vocab.order.size(), 0, 0}};
  while (!todo.empty() && !full) {
    const Span sp = todo.back();
    todo.pop_back();
    size_t i = sp.lo;
    auto len = [&](size_t k) { return vocab.byte_off[vocab.order[k] + 1] - vocab.byte_off[vocab.order[k]]; };
    while (i < sp.hi && len(i) == sp.depth) ++i;  // (tokens that end here come first in byte order)
    while (i < sp.hi) {
      const uint8_t c = vocab.bytes[vocab.byte_off[vocab.order[i]] + sp.depth];
      size_t j = i + 1;
      while (j < sp.hi && vocab.bytes[vocab.byte_off[vocab.order[j]] + sp.depth] == c) ++j;
      const int ns = trans(sp.state, c);
      if (ns >= 0) todo.push_back({i, j, sp.depth + 1, ns});
      i = j;
    }
  }
  if (full) return false;
  const int S = (int)cfg.size();
  out.n_states = S + 1;
  out.dead = S;
  out.start = 0;
  out.next.assign((size_t)(S + 1) * 256, (uint16_t)S);
  out.done.assign((size_t)S + 1, 0);
  for (int s = 0; s < S; ++s) {
    out.done[(size_t)s] = m.classify(cfg[(size_t)s]) == DONE;
    for (int c = 0; c < 256; ++c)
      if (next[(size_t)s][(size_t)c] >= 0) out.next[(size_t)s * 256 + (size_t)c] = (uint16_t)next[(size_t)s][(size_t)c];
  }
  return true;
}

inline bool Automaton::table(const Config& from, const Vocab& vocab, Table& out, int max_states) const {
  return build_table(*this, from, vocab, out, max_states);
}

}  // namespace jcon
}  // namespace arcinfer_b200

#include "json_automaton_step.hpp"
