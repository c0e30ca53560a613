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

namespace {
using arcinfer_b200::jcon::Automaton;
using arcinfer_b200::jcon::Config;

struct Jcon {
  std::unique_ptr<Automaton> au;
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

bool walk_text(const Jcon& j, const char* text, int64_t len, Config& st) {
  st = j.au->start();
  for (int64_t i = 0; i < len; ++i)
    if (!j.au->step(st, (uint8_t)text[i], false)) return false;
  return true;
}
}  // namespace

struct arcs_jcon {
  Jcon j;
};

extern "C" {

int arcs_jcon_create(const char* schema_json, int32_t object_only, const uint32_t* byte_off, const uint8_t* bytes,
                     int32_t V, arcs_jcon** out) {
  if (!schema_json || !out || V < 0 || (V > 0 && (!byte_off || (!bytes && byte_off[V] > 0)))) return ARCS_ERR_ARG;
  *out = nullptr;
  for (int32_t t = 0; t < V; ++t)
    if (byte_off[t + 1] < byte_off[t]) return ARCS_ERR_ARG;
  std::unique_ptr<arcs_jcon> h(new arcs_jcon);
  Jcon& j = h->j;
  j.au.reset(new Automaton(schema_json, object_only != 0));
  j.why = j.au->why_not();
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

int arcs_tcon_create(int32_t kind, const char* tools_json, const uint32_t* byte_off, const uint8_t* bytes, int32_t V, arcs_jcon** out) {
  if (!tools_json || !out || V < 0 || (V > 0 && (!byte_off || (!bytes && byte_off[V] > 0)))) return ARCS_ERR_ARG;
  *out = nullptr;
  if (kind != ARCS_TCON_GEMMA) return ARCS_ERR_UNSUPPORTED;  // (the Qwen form is served by the ranked head)
  for (int32_t t = 0; t < V; ++t)
    if (byte_off[t + 1] < byte_off[t]) return ARCS_ERR_ARG;
  std::unique_ptr<arcs_jcon> h(new arcs_jcon);
  Jcon& j = h->j;
  j.au.reset(new Automaton(tools_json, Automaton::GEMMA));
  j.why = j.au->why_not();
  if (V > 0) {
    j.byte_off.assign(byte_off, byte_off + V + 1);
    j.bytes.assign(bytes, bytes + byte_off[V]);
  } else {
    j.byte_off.assign(1, 0u);
  }
  j.vocab.reset(new Automaton::Vocab(j.byte_off.data(), j.bytes.data(), V));
  const bool ok = j.au->supported();
  *out = h.release();
  return ok ? ARCS_OK : ARCS_ERR_UNSUPPORTED;
}

const char* arcs_jcon_why(const arcs_jcon* h) { return h ? h->j.why.c_str() : "null handle"; }

int arcs_jcon_check(const arcs_jcon* h, const char* text, int64_t len) {
  if (!h || len < 0 || (len > 0 && !text) || !h->j.au->supported()) return -1;
  Config st;
  if (!walk_text(h->j, text, len, st)) return arcinfer_b200::jcon::FAIL;
  return h->j.au->classify(st);
}

int arcs_jcon_table(arcs_jcon* h, const char* text, int64_t len, const uint16_t** table, int32_t* n_states,
                    int32_t* dead, const uint8_t** done, int32_t* text_state) {
  if (!h || len < 0 || (len > 0 && !text) || !table || !n_states || !dead) return ARCS_ERR_ARG;
  Jcon& j = h->j;
  if (!j.au->supported()) return ARCS_ERR_UNSUPPORTED;
  Config st;
  const bool alive = walk_text(j, text, len, st);
  if (text_state) *text_state = alive ? j.au->classify(st) : arcinfer_b200::jcon::FAIL;
  if (!alive) return ARCS_ERR_ARG;  // (the answer so far is not a prefix of any match: no step follows it)
  const std::string key = arcinfer_b200::jcon::config_key(st);
  std::lock_guard<std::mutex> lock(j.mu);
  auto it = j.by_key.find(key);
  if (it != j.by_key.end()) {
    ++j.hits;
    j.lru.splice(j.lru.begin(), j.lru, it->second);
  } else {
    ++j.misses;
    j.lru.emplace_front();
    Jcon::Entry& e = j.lru.front();
    e.key = key;
    e.ok = j.au->table(st, *j.vocab, e.table);
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
