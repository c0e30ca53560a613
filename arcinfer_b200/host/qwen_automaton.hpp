// The Qwen 3.x tool-call form as an incremental machine (tcon::QwenCall::check,
// tools/tool_constraint.h:285-371): the text after <tool_call> is
//   <function=NAME> then <parameter=KEY> VALUE </parameter> blocks, </function> </tool_call>
// with up to two blanks (newline or space) between the parts. A value whose schema says "string"
// (or names no type) is raw text: anything without "</parameter>" or "<parameter="; a value of
// another type is JSON for its schema, checked by the JSON machine, and may be followed by one
// newline before "</parameter>".
//
// The reference finds the end of a value by searching the whole text for the markers and then
// parses the value again; here the markers are recognised as the bytes arrive (both begin with
// '<' and neither has a proper border, so a mismatch can only restart at a '<'). For a JSON value
// the bytes of a marker that is still being matched may yet turn out to belong to the value
// (a '<' inside a JSON string), so up to three readings of the value are carried at once, as the
// reference's search over the possible cuts does (:355-362): everything so far is value; the
// value ends before the marker being matched; it ends one newline earlier.
#pragma once
#include <map>
#include <memory>

#include "json_automaton.hpp"

namespace arcinfer_b200 {
namespace jcon {

class QwenAutomaton {
 public:
  enum Phase : uint8_t { Q_LEAD = 0, Q_NAME, Q_BETWEEN, Q_MARK, Q_KEY, Q_VAL_START, Q_RAW, Q_JSON, Q_TAIL, Q_END };
  struct State {
    uint8_t phase = Q_LEAD;
    uint8_t ws = 0;        // blanks of the current gap
    uint8_t which = 0;     // value: the marker being matched: 0 either ("<"), 1 "</parameter>", 2 "<parameter="
    uint8_t nl = 0;        // JSON value: the byte before the marker being matched (or the last byte) is a newline
    uint8_t other = 0;     // a key the schema does not name was closed during a table walk
    int32_t n = 0;         // position in the literal, or bytes of the marker matched
    int32_t tool = -1;
    int32_t sub = -1;      // JSON value: which value machine
    std::string text;      // name, key, or the part of a marker seen
    std::vector<std::string> seen;  // keys used, sorted
    // JSON value: the three readings (empty: that reading has failed)
    Config all, cut, cut_nl;
  };

  explicit QwenAutomaton(const std::string& tools_json) {
    if (!JVal::parse(tools_json, doc_)) {
      why_ = "the tool list is not JSON";
      return;
    }
    supported_ = true;
    for (const JVal& t : doc_.a) {  // tools/tool_constraint.h:45-51
      const JVal& f = t.has("function") ? t["function"] : t;
      if (f["name"].str().empty()) continue;
      tools_.push_back({f["name"].str(), f["parameters"].is_object() ? &f["parameters"] : &empty_object()});
    }
    // a machine for every value schema that is checked as JSON (:350, :355-368)
    for (size_t ti = 0; ti < tools_.size(); ++ti) {
      const JVal& params = *tools_[ti].second;
      for (const auto& kv : params["properties"].o) add_value_machine(&kv.second);
      if (params["additionalProperties"].is_object()) add_value_machine(&params["additionalProperties"]);
    }
  }
  bool supported() const { return supported_; }
  const std::string& why_not() const { return why_; }

  State start() const { return State(); }
  Res classify(const State& st) const { return st.phase == Q_END ? DONE : PARTIAL; }
  Res check(const std::string& text) const {
    State st = start();
    for (unsigned char ch : text)
      if (!step(st, ch, false)) return FAIL;
    return classify(st);
  }
  std::string key(const State& st) const {
    std::string k;
    const uint8_t head[6] = {st.phase, st.ws, st.which, st.nl, st.other, 0};
    k.append(reinterpret_cast<const char*>(head), 6);
    k.append(reinterpret_cast<const char*>(&st.n), 4);
    k.append(reinterpret_cast<const char*>(&st.tool), 4);
    k.append(reinterpret_cast<const char*>(&st.sub), 4);
    auto put = [&](const std::string& x) {
      const uint32_t l = (uint32_t)x.size();
      k.append(reinterpret_cast<const char*>(&l), 4);
      k += x;
    };
    put(st.text);
    const uint32_t ns = (uint32_t)st.seen.size();
    k.append(reinterpret_cast<const char*>(&ns), 4);
    for (const std::string& x : st.seen) put(x);
    put(config_key(st.all));
    put(config_key(st.cut));
    put(config_key(st.cut_nl));
    return k;
  }

  bool step(State& st, uint8_t c, bool walk) const {
    static const std::string kFn = "<function=", kParam = "<parameter=", kEndFn = "</function>", kEndParam = "</parameter>", kEndCall = "</tool_call>";
    auto blank = [](uint8_t x) { return x == '\n' || x == ' '; };
    switch (st.phase) {
      case Q_LEAD:  // :293: up to two blanks, then "<function="
        if (st.n == 0 && blank(c) && st.ws < 2) {
          ++st.ws;
          return true;
        }
        if (c != (uint8_t)kFn[(size_t)st.n]) return false;
        if (++st.n == (int32_t)kFn.size()) {
          st.phase = Q_NAME;
          st.text.clear();
        }
        return true;
      case Q_NAME: {  // :294-301
        if (c == '\n') return false;
        if (c != '>') {
          st.text.push_back((char)c);
          for (const auto& t : tools_)
            if (t.first.compare(0, st.text.size(), st.text) == 0) return true;
          return false;
        }
        st.tool = -1;
        for (size_t i = 0; i < tools_.size(); ++i)
          if (tools_[i].first == st.text) st.tool = (int32_t)i;  // (the last of that name, :54-61)
        if (st.tool < 0) return false;
        return between(st);
      }
      case Q_BETWEEN:  // :308-318: up to two blanks, then a marker
        if (blank(c) && st.ws < 2) {
          ++st.ws;
          return true;
        }
        if (c != '<') return false;
        st.phase = Q_MARK;
        st.text = "<";
        return true;
      case Q_MARK: {  // "<parameter=" or "</function>" (:313-326)
        st.text.push_back((char)c);
        const bool p = kParam.compare(0, st.text.size(), st.text) == 0, f = kEndFn.compare(0, st.text.size(), st.text) == 0;
        if (!p && !f) return false;
        if (!p && st.text.size() == 2) {  // the end of the function: only with every required parameter (:320-322)
          for (const JVal& q : params(st)["required"].a)
            if (!std::binary_search(st.seen.begin(), st.seen.end(), q.str())) return false;
        }
        if (p && st.text.size() == kParam.size()) {
          st.phase = Q_KEY;
          st.text.clear();
          // (:341: a parameter can begin only where some key can still follow)
          const JVal& ps = params(st);
          if (!key_ok(st, ps, Automaton::any_key_of_public(ps), true)) return false;
        } else if (f && st.text.size() == kEndFn.size()) {
          st.phase = Q_TAIL;  // :325: up to two blanks, then "</tool_call>", then nothing
          st.text.clear();
          st.ws = 0;
          st.n = 0;
        }
        return true;
      }
      case Q_KEY: {  // :328-346
        if (c == '\n') return false;
        const JVal& ps = params(st);
        const bool any_key = Automaton::any_key_of_public(ps);
        if (c != '>') {
          if (st.text == kOtherKey) return true;
          st.text.push_back((char)c);
          if (!key_ok(st, ps, any_key, true)) return false;
          if (walk && any_key) {  // fold a key no property and no used key begins with
            bool known = false;
            for (const auto& kv : ps["properties"].o) known = known || kv.first.compare(0, st.text.size(), st.text) == 0;
            for (const std::string& k : st.seen) known = known || k.compare(0, st.text.size(), st.text) == 0;
            if (!known) st.text = kOtherKey;
          }
          return true;
        }
        const JVal* vs = nullptr;
        if (st.text == kOtherKey) {
          if (!any_key || st.other) return false;  // (a second such key in one walk cannot be told from the first)
          st.other = 1;
        } else {
          if (!key_ok(st, ps, any_key, false)) return false;
          st.seen.insert(std::upper_bound(st.seen.begin(), st.seen.end(), st.text), st.text);
          if (!ps["properties"][st.text].is_null()) vs = &ps["properties"][st.text];
        }
        if (!vs && ps["additionalProperties"].is_object()) vs = &ps["additionalProperties"];  // :351
        st.text.clear();
        st.n = 0;
        st.which = 0;
        st.nl = 0;
        st.sub = -1;
        const bool is_str = vs && (*vs)["type"].is_string() && (*vs)["type"].s == "string";
        if (vs && !is_str && vs->has("type")) {
          st.sub = machines_.at(vs);
          st.all = st.cut = subs_[(size_t)st.sub]->start();
          st.cut_nl.clear();
        }
        st.phase = Q_VAL_START;
        return true;
      }
      case Q_VAL_START:  // :347: one newline right after the '>' is not part of the value
        st.phase = st.sub >= 0 ? Q_JSON : Q_RAW;
        if (c == '\n') return true;
        return step(st, c, walk);
      case Q_RAW:  // :348-353, :364-369: any text up to "</parameter>", without "<parameter="
        if (!marker(st, c)) return false;
        if (st.which == 1 && st.n == (int32_t)kEndParam.size()) return between(st);
        return true;
      case Q_JSON: {
        const Automaton& au = *subs_[(size_t)st.sub];
        const int32_t held = st.n;  // bytes of a marker matched before this one
        if (!marker(st, c)) return false;
        if (st.n > held) {  // the marker goes on (or begins): only the "all is value" reading takes the byte
          if (!st.all.empty() && !au.step(st.all, c, false)) st.all.clear();
          if (st.which == 1 && st.n == (int32_t)kEndParam.size()) {
            // the value is what came before the marker, less one newline (:364-367), and must be complete
            const Config& v = st.nl ? st.cut_nl : st.cut;
            if (v.empty() || au.classify(v) != DONE) return false;
            st.all.clear();
            st.cut.clear();
            st.cut_nl.clear();
            return between(st);
          }
        } else {  // no marker after all: what was held is value, and so is this byte (unless it begins a marker)
          st.cut = st.all;
          st.nl = 0;
          st.cut_nl.clear();
          if (st.n == 0) {
            if (c == '\n') {
              st.cut_nl = st.cut;
              st.nl = 1;
            }
            if (!st.cut.empty() && !au.step(st.cut, c, false)) st.cut.clear();
            st.all = st.cut;
          } else {  // c == '<': held again
            if (!st.all.empty() && !au.step(st.all, c, false)) st.all.clear();
          }
        }
        // :355-362: some reading must still stand. "Before the marker" readings count only while
        // the held bytes can still become "</parameter>".
        const bool cut_ok = st.which != 2;
        return !st.all.empty() || (cut_ok && !st.cut.empty()) || (cut_ok && st.nl && !st.cut_nl.empty());
      }
      case Q_TAIL:
        if (st.n == 0 && blank(c) && st.ws < 2) {
          ++st.ws;
          return true;
        }
        if (c != (uint8_t)kEndCall[(size_t)st.n]) return false;
        if (++st.n == (int32_t)kEndCall.size()) st.phase = Q_END;
        return true;
      default:  // Q_END: nothing may follow (:326)
        return false;
    }
  }

 private:
  JVal doc_;
  bool supported_ = false;
  std::string why_;
  std::vector<std::pair<std::string, const JVal*>> tools_;
  std::map<const JVal*, int> machines_;
  std::vector<std::unique_ptr<Automaton>> subs_;

  static const JVal& empty_object() {
    static const JVal o = [] {
      JVal v;
      v.t = JVal::Object;
      return v;
    }();
    return o;
  }
  const JVal& params(const State& st) const { return *tools_[(size_t)st.tool].second; }
  void add_value_machine(const JVal* vs) {
    const bool is_str = (*vs)["type"].is_string() && (*vs)["type"].s == "string";
    if (is_str || !vs->has("type") || machines_.count(vs)) return;
    subs_.emplace_back(new Automaton(vs->dump(), false));  // jcon::Checker(vs, false): the value's schema is its own root
    machines_[vs] = (int)subs_.size() - 1;
    if (!subs_.back()->supported()) {
      supported_ = false;
      why_ = subs_.back()->why_not();
    }
  }
  bool between(State& st) const {
    st.phase = Q_BETWEEN;
    st.ws = 0;
    st.n = 0;
    st.which = 0;
    st.text.clear();
    return true;
  }
  // :330-340
  static bool key_ok(const State& st, const JVal& ps, bool any_key, bool pre) {
    if (std::binary_search(st.seen.begin(), st.seen.end(), st.text) && !pre) return false;
    if (any_key) return !st.text.empty() || pre;
    for (const auto& kv : ps["properties"].o) {
      if (std::binary_search(st.seen.begin(), st.seen.end(), kv.first)) continue;
      if (pre ? kv.first.compare(0, st.text.size(), st.text) == 0 : kv.first == st.text) return true;
    }
    return false;
  }
  // One byte of a value through the marker matcher (st.which, st.n). false: "<parameter=" came
  // before "</parameter>" (:349-350).
  static bool marker(State& st, uint8_t c) {
    static const std::string kParam = "<parameter=", kEndParam = "</parameter>";
    if (st.n > 0) {
      const bool a = st.which != 2 && (size_t)st.n < kEndParam.size() && c == (uint8_t)kEndParam[(size_t)st.n];
      const bool b = st.which != 1 && (size_t)st.n < kParam.size() && c == (uint8_t)kParam[(size_t)st.n];
      if (a || b) {
        st.which = a ? 1 : 2;  // (they part at their second byte)
        ++st.n;
        return !(st.which == 2 && st.n == (int32_t)kParam.size());
      }
    }
    st.which = 0;
    st.n = c == '<' ? 1 : 0;
    return true;
  }
};

}  // namespace jcon
}  // namespace arcinfer_b200
