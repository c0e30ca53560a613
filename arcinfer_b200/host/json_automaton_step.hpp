// The transitions of the JSON automaton (included by json_automaton.hpp): one byte at a time
// through the frames that restate tools/json_constraint.h.
#pragma once

namespace arcinfer_b200 {
namespace jcon {

// :209-225 allowed(k, prefix): may the key (or key prefix) k be written into this object now?
inline bool Automaton::key_allowed(const Frame& obj, const std::string& k, bool prefix) const {
  const JVal& sc = node(obj.node);
  const bool used = std::binary_search(obj.seen.begin(), obj.seen.end(), k);
  if (used && !prefix) return false;
  if (any_key_of(sc)) return true;
  for (const auto& kv : sc["properties"].o) {
    if (std::binary_search(obj.seen.begin(), obj.seen.end(), kv.first)) continue;
    if (prefix ? kv.first.compare(0, k.size(), k) == 0 : kv.first == k) return true;
  }
  return false;
}

// A value of schema `node` at nesting `depth` starts with byte c (tools/json_constraint.h:92-133).
inline bool Automaton::start_value(Config& st, int node_idx, int depth, uint8_t c) const {
  if (depth > 32) return false;                                             // :93
  const JVal& root = root_of(st);
  const JVal& sc = resolve(node(node_idx), root);
  if (const JVal* alt = alternatives(sc)) {                                 // :96-108 (branches told apart by c, see vet)
    for (const JVal& br : alt->a) {
      std::vector<const JVal*> path;
      if (first_chars(br, path, root).has(c)) return start_value(st, node_id(&br), depth + 1, c);
    }
    return false;
  }
  Frame f;
  f.node = node_id(&sc);
  f.depth = depth;
  if (is_enum(sc)) {                                                        // :112-124
    f.type = F_ENUM;
    st.push_back(f);
    return step(st, c);
  }
  if (c == '{') {
    if (!has_type(sc, "object")) return false;
    f.type = dialect_ == GEMMA ? F_GOBJ : F_OBJ;
    f.sub = dialect_ == GEMMA ? (uint8_t)GO_OPEN : (uint8_t)O_OPEN;
    st.push_back(f);
    return true;
  }
  if (dialect_ == GEMMA && c == '<') {  // tools/tool_constraint.h:162, :183-190: <|"|> text <|"|>
    if (!has_type(sc, "string")) return false;
    f.type = F_GSTR;
    f.sub = GS_OPEN;
    f.node = -1;
    f.n = 1;
    st.push_back(f);
    return true;
  }
  if (c == '[') {
    if (!has_type(sc, "array")) return false;
    f.type = F_ARR;
    f.sub = A_OPEN;
    st.push_back(f);
    return true;
  }
  if (c == '"' && dialect_ == JSON) {
    if (!has_type(sc, "string")) return false;
    f.type = F_STR;
    f.node = -1;
    st.push_back(f);
    return true;
  }
  if (c == '-' || (c >= '0' && c <= '9')) {
    if (!has_type(sc, "number")) return false;
    f.type = F_NUM;
    f.flag = integer_only(sc);
    f.node = -1;
    f.sub = c == '-' ? N_MINUS : c == '0' ? N_ZERO : N_INT;
    st.push_back(f);
    return true;
  }
  if (c == 't' || c == 'f' || c == 'n') {
    if (!has_type(sc, c == 'n' ? "null" : "boolean")) return false;
    f.type = F_LIT;
    f.node = -1;
    f.text = c == 't' ? "true" : c == 'f' ? "false" : "null";
    f.n = 1;
    st.push_back(f);
    return true;
  }
  return false;
}

// The value (or key) on top of the stack is complete: pop it and tell the frame below.
inline bool Automaton::complete(Config& st, bool walk) const {
  Frame done = std::move(st.back());
  st.pop_back();
  Frame& p = st.back();
  if (p.type == F_TOP) {
    p.sub = dialect_ == GEMMA ? (uint8_t)G_CLOSE : (uint8_t)T_TRAIL;  // (GEMMA: the close marker follows, :93)
    p.ws = 0;
    p.n = 0;
    return true;
  }
  if (p.type == F_GOBJ) {
    p.sub = GO_AFTER_VALUE;
    return true;
  }
  if (p.type == F_ARR) {
    const JVal& sc = node(p.node);
    const int64_t mn = sc["minItems"].as_int(0), mx = sc["maxItems"].as_int(1 << 30);
    const int64_t cap = mx >= (1 << 30) ? mn : std::max(mn, mx);  // (beyond it one more element changes nothing)
    p.n = (int32_t)std::min<int64_t>((int64_t)p.n + 1, std::max<int64_t>(cap, 1));
    p.sub = A_AFTER_ELEM;
    p.ws = 0;
    return true;
  }
  // F_OBJ
  if (p.sub == O_IN_KEY) {  // :227-229: the key is complete
    const bool folded = done.text == kOtherKey;
    if (folded) {
      // (a key no property and no used key starts with: allowed only where other keys are, and a
      //  second such key closed in the same object during one walk cannot be told from the first)
      if (!any_key_of(node(p.node)) || p.flag) return false;
      p.flag = 1;
    } else {
      if (!key_allowed(p, done.text, false)) return false;
      p.seen.insert(std::upper_bound(p.seen.begin(), p.seen.end(), done.text), done.text);
    }
    p.text = done.text;  // (the value's schema is looked up under it)
    p.sub = O_AFTER_KEY;
    p.ws = 0;
    (void)walk;
    return true;
  }
  p.sub = O_AFTER_VALUE;
  p.ws = 0;
  return true;
}

inline bool Automaton::step(Config& st, uint8_t c, bool walk) const {
  for (;;) {  // (a number ends before the byte that follows it: that byte is then given to the frame below)
    Frame& f = st.back();
    switch (f.type) {
      case F_TOP:
        if (dialect_ == GEMMA) return step_gemma_top(st, c);
        if (f.sub == T_LEAD) {                               // :38-41
          if (is_ws(c)) return true;
          if (object_only_ && c != '{') return false;
          f.sub = T_VALUE;
          return start_value(st, node_id(&root_), 0, c);
        }
        if (f.sub == T_TRAIL) return is_ws(c) && ++f.ws <= 2;  // :44-46
        return false;
      case F_LIT:                                            // :135-142
        if (c != (uint8_t)f.text[(size_t)f.n]) return false;
        if (++f.n == (int32_t)f.text.size()) return complete(st, walk);
        return true;
      case F_NUM: {                                          // :143-168
        const bool digit = c >= '0' && c <= '9';
        switch (f.sub) {
          case N_MINUS:
            if (c == '0') f.sub = N_ZERO;
            else if (c >= '1' && c <= '9') f.sub = N_INT;
            else return false;
            return true;
          case N_INT:
            if (digit) return true;
            [[fallthrough]];
          case N_ZERO:
            if (c == '.') {
              if (f.flag) return false;
              f.sub = N_DOT;
              return true;
            }
            if ((c == 'e' || c == 'E') && dialect_ == JSON) {  // (the Gemma form has no exponent, tools/tool_constraint.h:191-208)
              if (f.flag) return false;
              f.sub = N_E;
              return true;
            }
            break;  // the number is complete
          case N_DOT:
            if (!digit) return false;
            f.sub = N_FRAC;
            return true;
          case N_FRAC:
            if (digit) return true;
            if ((c == 'e' || c == 'E') && dialect_ == JSON) {
              f.sub = N_E;
              return true;
            }
            break;
          case N_E:
            if (c == '+' || c == '-') {
              f.sub = N_ESIGN;
              return true;
            }
            [[fallthrough]];
          case N_ESIGN:
            if (!digit) return false;
            f.sub = N_EXP;
            return true;
          case N_EXP:
            if (digit) return true;
            break;
        }
        if (!complete(st, walk)) return false;
        continue;  // c goes to the frame below
      }
      case F_STR:                                            // :170-198
        if (f.sub == S_NORMAL) {
          if (c == '"') return complete(st, walk);
          if (c < 0x20) return false;
          if (c == '\\') {
            f.sub = S_ESC;
            return true;
          }
          if (f.flag) f.text.push_back((char)c);
        } else if (f.sub == S_ESC) {
          if (c == 'u') {
            f.sub = S_HEX;
            f.n = 4;
            return true;
          }
          // (c == 0 passes, as it does in the reference, whose strchr finds the terminator: :187)
          if (!std::strchr("\"\\/bfnrt", (char)c)) return false;
          f.sub = S_NORMAL;
          if (f.flag) f.text.push_back(c == 'n' ? '\n' : c == 't' ? '\t' : (char)c);
        } else {  // S_HEX
          const bool hex = (c >= '0' && c <= '9') || (c >= 'a' && c <= 'f') || (c >= 'A' && c <= 'F');
          if (!hex) return false;
          if (--f.n > 0) return true;
          f.sub = S_NORMAL;
          if (f.flag) f.text.push_back('?');
        }
        if (f.flag) {  // a key: it must stay (a prefix of) a key the object can take (:230)
          const Frame& obj = st[st.size() - 2];
          if (f.text != kOtherKey) {
            if (!key_allowed(obj, f.text, true)) return false;
            if (walk && any_key_of(node(obj.node))) {
              // fold: no property and no used key starts with this text, so all that can be said of
              // it later is that it is "another key"
              bool prefix_of_known = false;
              for (const auto& kv : node(obj.node)["properties"].o) prefix_of_known = prefix_of_known || kv.first.compare(0, f.text.size(), f.text) == 0;
              for (const std::string& k : obj.seen) prefix_of_known = prefix_of_known || k.compare(0, f.text.size(), f.text) == 0;
              if (!prefix_of_known) f.text = kOtherKey;
            }
          }
        }
        return true;
      case F_ENUM: {                                         // :112-124
        f.text.push_back((char)c);
        bool partial = false;
        for (const std::string& o : options(node(f.node))) {
          if (o == f.text) return complete(st, walk);
          if (o.size() > f.text.size() && o.compare(0, f.text.size(), f.text) == 0) partial = true;
        }
        return partial;
      }
      case F_OBJ: {                                          // :199-255
        const JVal& sc = node(f.node);
        if (is_ws(c)) return f.sub != O_IN_KEY && f.sub != O_IN_VALUE && ++f.ws <= 8;  // :66-70
        switch (f.sub) {
          case O_AFTER_VALUE:
            if (c == ',') {                                  // :238-241: a comma only where another key can follow
              bool more = any_key_of(sc);
              for (const auto& kv : sc["properties"].o) more = more || !std::binary_search(f.seen.begin(), f.seen.end(), kv.first);
              if (!more) return false;
              f.sub = O_AFTER_COMMA;
              f.ws = 0;
              return true;
            }
            [[fallthrough]];
          case O_OPEN:
            if (c == '}') {                                  // :233-236
              for (const JVal& r : sc["required"].a)
                if (!std::binary_search(f.seen.begin(), f.seen.end(), r.str())) return false;
              return complete(st, walk);
            }
            if (f.sub == O_AFTER_VALUE) return false;
            [[fallthrough]];
          case O_AFTER_COMMA: {
            if (c != '"') return false;                      // :246
            f.sub = O_IN_KEY;
            Frame k;
            k.type = F_STR;
            k.flag = 1;
            st.push_back(k);
            return key_allowed(st[st.size() - 2], std::string(), true);
          }
          case O_AFTER_KEY:
            if (c != ':') return false;                      // :235
            f.sub = O_AFTER_COLON;
            f.ws = 0;
            return true;
          case O_AFTER_COLON: {                              // :250-253
            const JVal& props = sc["properties"];
            const JVal& addl = sc["additionalProperties"];
            const JVal* vs = f.text == kOtherKey || props[f.text].is_null() ? (addl.is_object() ? &addl : nullptr) : &props[f.text];
            f.sub = O_IN_VALUE;
            const int depth = f.depth;
            return start_value(st, vs ? node_id(vs) : -1, depth + 1, c);
          }
          default:
            return false;
        }
      }
      case F_ARR: {                                          // :256-281
        const JVal& sc = node(f.node);
        if (is_ws(c) && dialect_ == JSON) return f.sub != A_IN_VALUE && ++f.ws <= 8;
        const int64_t mn = sc["minItems"].as_int(0), mx = sc["maxItems"].as_int(1 << 30);
        if (c == ']' && (f.sub == A_OPEN || f.sub == A_AFTER_ELEM)) {
          if (f.n < mn) return false;
          return complete(st, walk);
        }
        if (f.sub == A_AFTER_ELEM) {
          if (c != ',') return false;
          f.sub = A_AFTER_COMMA;
          f.ws = 0;
          return true;
        }
        if (f.sub != A_OPEN && f.sub != A_AFTER_COMMA) return false;
        if (f.n >= mx) return false;                         // :274
        f.sub = A_IN_VALUE;
        const int depth = f.depth;
        const JVal* items = sc["items"].is_object() ? &sc["items"] : nullptr;
        return start_value(st, items ? node_id(items) : -1, depth + 1, c);
      }
      case F_GSTR:                                           // tools/tool_constraint.h:183-190
        if (f.sub == GS_OPEN) {
          if (c != (uint8_t)kGemmaQuote[f.n]) return false;
          if (++f.n == 5) {
            f.sub = GS_BODY;
            f.n = 0;
          }
          return true;
        }
        // any text up to the first closing delimiter (no proper border in <|"|>: after a mismatch
        // only a '<' can begin it again)
        if (c == (uint8_t)kGemmaQuote[f.n]) {
          if (++f.n == 5) return complete(st, walk);
        } else {
          f.n = c == '<' ? 1 : 0;
        }
        return true;
      case F_GOBJ:
        return step_gemma_object(st, c, walk);
      default:
        return false;
    }
  }
}

// call:NAME{...}<tool_call|> (tools/tool_constraint.h:79-94)
inline bool Automaton::step_gemma_top(Config& st, uint8_t c) const {
  Frame& f = st.back();
  switch (f.sub) {
    case G_CALL:
      if (c != (uint8_t)"call:"[f.n]) return false;
      if (++f.n == 5) {
        f.sub = G_NAME;
        f.text.clear();
      }
      return true;
    case G_NAME: {
      if (c != '{') {  // :84-88: the name so far must begin some tool's name
        f.text.push_back((char)c);
        for (const auto& t : tools_)
          if (t.first.compare(0, f.text.size(), f.text) == 0) return true;
        return false;
      }
      const JVal* params = nullptr;  // :54-61: the last tool of that name
      for (const auto& t : tools_)
        if (t.first == f.text) params = t.second;
      if (!params) return false;
      f.node = node_id(params);  // (what $ref is resolved against from here on)
      f.text.clear();
      f.sub = T_VALUE;
      const JVal& sc = resolve(*params, *params);
      if (alternatives(sc)) return start_value(st, node_id(params), 0, c);  // :133-147 come before the "always an object" of :149
      Frame o;
      o.type = F_GOBJ;
      o.sub = GO_OPEN;
      o.node = node_id(&sc);
      o.depth = 0;
      st.push_back(o);
      return true;
    }
    case G_CLOSE:
      if (c != (uint8_t)kGemmaClose[f.n]) return false;
      if (++f.n == (int32_t)std::strlen(kGemmaClose)) f.sub = G_END;
      return true;
    default:  // G_END: nothing may follow (:94); T_VALUE: a value frame is on top, not this one
      return false;
  }
}

// {key:value,...} with bare keys and no whitespace (tools/tool_constraint.h:209-257)
inline bool Automaton::step_gemma_object(Config& st, uint8_t c, bool walk) const {
  Frame& f = st.back();
  const JVal& sc = node(f.node);
  auto closes = [&]() {  // :222-226
    for (const JVal& r : sc["required"].a)
      if (!std::binary_search(f.seen.begin(), f.seen.end(), r.str())) return false;
    return complete(st, walk);
  };
  const bool key_char = std::isalnum(c) || c == '_' || c == '-' || c == '.' || c == '$';  // :234
  switch (f.sub) {
    case GO_OPEN:
      if (c == '}') return closes();
      f.sub = GO_KEY;
      f.text.clear();
      [[fallthrough]];
    case GO_KEY:
      if (key_char) {
        if (f.text != kOtherKey) {
          f.text.push_back((char)c);
          if (!key_allowed(f, f.text, true)) return false;  // :236-247 with prefix
          if (walk && any_key_of(sc)) {  // fold, as for JSON keys
            bool prefix_of_known = false;
            for (const auto& kv : sc["properties"].o) prefix_of_known = prefix_of_known || kv.first.compare(0, f.text.size(), f.text) == 0;
            for (const std::string& k : f.seen) prefix_of_known = prefix_of_known || k.compare(0, f.text.size(), f.text) == 0;
            if (!prefix_of_known) f.text = kOtherKey;
          }
        }
        return true;
      }
      if (c != ':') return false;  // :249
      if (f.text == kOtherKey) {
        if (!any_key_of(sc) || f.flag) return false;
        f.flag = 1;
      } else {
        if (f.text.empty() || !key_allowed(f, f.text, false)) return false;
        f.seen.insert(std::upper_bound(f.seen.begin(), f.seen.end(), f.text), f.text);
      }
      f.sub = GO_AFTER_COLON;
      return true;
    case GO_AFTER_COLON: {  // :251-255
      const JVal& props = sc["properties"];
      const JVal& addl = sc["additionalProperties"];
      const JVal* vs = f.text == kOtherKey || props[f.text].is_null() ? (addl.is_object() ? &addl : nullptr) : &props[f.text];
      f.sub = GO_IN_VALUE;
      const int depth = f.depth;
      return start_value(st, vs ? node_id(vs) : -1, depth + 1, c);
    }
    case GO_AFTER_VALUE:
      if (c == '}') return closes();
      if (c != ',') return false;  // :228
      {
        bool more = any_key_of(sc);  // :229: a comma only where another key can follow
        for (const auto& kv : sc["properties"].o) more = more || !std::binary_search(f.seen.begin(), f.seen.end(), kv.first);
        if (!more) return false;
      }
      f.sub = GO_KEY;
      f.text.clear();
      return true;
    default:
      return false;
  }
}

}  // namespace jcon
}  // namespace arcinfer_b200
