// C ABI of the JSON-constraint bridge: a schema and a vocabulary in, the [S][256] byte table that
// arcs_dfa_mask walks out. Host code only (no kernel in this file): it replaces the calls
// jc->check(ans + piece(t)) != FAIL that tools/server_chat.h:553-557 makes per candidate token,
// and jc->check(ans) == DONE of :550, by one table per decoding step.
#include <cstring>
#include <list>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>

#include "../../include/arcsample.h"
#include "../host/json_automaton.hpp"
#include "../host/qwen_automaton.hpp"

namespace {
using arcinfer_b200::jcon::Automaton;
using arcinfer_b200::jcon::QwenAutomaton;

// what a handle needs of a machine, whatever its state type
struct Machine {
  virtual ~Machine() = default;
  virtual bool supported() const = 0;
  virtual std::string why() const = 0;
  // walks the text: false when it fails; cls: PARTIAL / DONE; key: the configuration reached
  virtual bool walk(const char* text, int64_t len, int& cls, std::string* key) = 0;
  // the table from the configuration of the last walk
  virtual bool table(const Automaton::Vocab& vocab, Automaton::Table& out) = 0;
};
template <class M>
struct MachineOf : Machine {
  M m;
  typename M::State at;
  template <class... A>
  explicit MachineOf(A&&... a) : m(std::forward<A>(a)...) {}
  bool supported() const override { return m.supported(); }
  std::string why() const override { return m.why_not(); }
  bool walk(const char* text, int64_t len, int& cls, std::string* key) override {
    at = m.start();
    for (int64_t i = 0; i < len; ++i)
      if (!m.step(at, (uint8_t)text[i], false)) return false;
    cls = m.classify(at);
    if (key) *key = m.key(at);
    return true;
  }
  bool table(const Automaton::Vocab& vocab, Automaton::Table& out) override { return arcinfer_b200::jcon::build_table(m, at, vocab, out, 8192); }
};

struct Jcon {
  std::unique_ptr<Machine> au;
  std::vector<uint32_t> byte_off;
  std::vector<uint8_t> bytes;
  std::unique_ptr<Automaton::Vocab> vocab;
  std::string why;
  // tables by configuration, least recently used last: a decoding spends most of its steps in a few
  // configurations (inside a string, between two digits), whose tables are built once
  struct Entry {
    std::string key;
    Automaton::Table table;
    bool ok;
  };
  std::list<Entry> lru;
  std::unordered_map<std::string, std::list<Entry>::iterator> by_key;
  size_t max_entries = 256;
  int64_t hits = 0, misses = 0;
  std::mutex mu;
};

int make_handle(std::unique_ptr<Machine> m, const uint32_t* byte_off, const uint8_t* bytes, int32_t V, struct arcs_jcon** out);
}  // namespace

struct arcs_jcon {
  Jcon j;
};

namespace {
int make_handle(std::unique_ptr<Machine> m, const uint32_t* byte_off, const uint8_t* bytes, int32_t V, arcs_jcon** out) {
  for (int32_t t = 0; t < V; ++t)
    if (byte_off[t + 1] < byte_off[t]) return ARCS_ERR_ARG;
  std::unique_ptr<arcs_jcon> h(new arcs_jcon);
  Jcon& j = h->j;
  j.au = std::move(m);
  j.why = j.au->why();
  if (V > 0) {
    j.byte_off.assign(byte_off, byte_off + V + 1);
    j.bytes.assign(bytes, bytes + byte_off[V]);
  } else {
    j.byte_off.assign(1, 0u);
  }
  j.vocab.reset(new Automaton::Vocab(j.byte_off.data(), j.bytes.data(), V));
  const bool ok = j.au->supported();
  *out = h.release();  // (kept also when unsupported, so that arcs_jcon_why can say why)
  return ok ? ARCS_OK : ARCS_ERR_UNSUPPORTED;
}
}  // namespace

extern "C" {

int arcs_jcon_create(const char* schema_json, int32_t object_only, const uint32_t* byte_off, const uint8_t* bytes,
                     int32_t V, arcs_jcon** out) {
  if (!schema_json || !out || V < 0 || (V > 0 && (!byte_off || (!bytes && byte_off[V] > 0)))) return ARCS_ERR_ARG;
  *out = nullptr;
  return make_handle(std::unique_ptr<Machine>(new MachineOf<Automaton>(std::string(schema_json), object_only != 0)), byte_off, bytes, V, out);
}

int arcs_tcon_create(int32_t kind, const char* tools_json, const uint32_t* byte_off, const uint8_t* bytes, int32_t V, arcs_jcon** out) {
  if (!tools_json || !out || V < 0 || (V > 0 && (!byte_off || (!bytes && byte_off[V] > 0)))) return ARCS_ERR_ARG;
  *out = nullptr;
  if (kind == ARCS_TCON_GEMMA)
    return make_handle(std::unique_ptr<Machine>(new MachineOf<Automaton>(std::string(tools_json), Automaton::GEMMA)), byte_off, bytes, V, out);
  if (kind == ARCS_TCON_QWEN) return make_handle(std::unique_ptr<Machine>(new MachineOf<QwenAutomaton>(std::string(tools_json))), byte_off, bytes, V, out);
  return ARCS_ERR_ARG;
}

const char* arcs_jcon_why(const arcs_jcon* h) { return h ? h->j.why.c_str() : "null handle"; }

int arcs_jcon_check(const arcs_jcon* h, const char* text, int64_t len) {
  if (!h || len < 0 || (len > 0 && !text) || !h->j.au->supported()) return -1;
  Jcon& j = const_cast<arcs_jcon*>(h)->j;
  std::lock_guard<std::mutex> lock(j.mu);
  int cls = 0;
  if (!j.au->walk(text, len, cls, nullptr)) return arcinfer_b200::jcon::FAIL;
  return cls;
}

int arcs_jcon_table(arcs_jcon* h, const char* text, int64_t len, const uint16_t** table, int32_t* n_states,
                    int32_t* dead, const uint8_t** done, int32_t* text_state) {
  if (!h || len < 0 || (len > 0 && !text) || !table || !n_states || !dead) return ARCS_ERR_ARG;
  Jcon& j = h->j;
  if (!j.au->supported()) return ARCS_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(j.mu);
  int cls = 0;
  std::string key;
  const bool alive = j.au->walk(text, len, cls, &key);
  if (text_state) *text_state = alive ? cls : arcinfer_b200::jcon::FAIL;
  if (!alive) return ARCS_ERR_ARG;  // (the answer so far is not a prefix of any match: no step follows it)
  auto it = j.by_key.find(key);
  if (it != j.by_key.end()) {
    ++j.hits;
    j.lru.splice(j.lru.begin(), j.lru, it->second);
  } else {
    ++j.misses;
    j.lru.emplace_front();
    Jcon::Entry& e = j.lru.front();
    e.key = key;
    e.ok = j.au->table(*j.vocab, e.table);
    j.by_key[key] = j.lru.begin();
    if (j.lru.size() > j.max_entries) {
      j.by_key.erase(j.lru.back().key);
      j.lru.pop_back();
    }
  }
  const Jcon::Entry& e = j.lru.front();
  if (!e.ok) return ARCS_ERR_UNSUPPORTED;
  *table = e.table.next.data();
  *n_states = e.table.n_states;
  *dead = e.table.dead;
  if (done) *done = e.table.done.data();
  return ARCS_OK;
}

void arcs_jcon_cache_stats(const arcs_jcon* h, int64_t* hits, int64_t* misses) {
  if (!h) return;
  if (hits) *hits = h->j.hits;
  if (misses) *misses = h->j.misses;
}

void arcs_jcon_destroy(arcs_jcon* h) { delete h; }

}  // extern "C"
