// Entry points that are not tied to one kernel: version, error text, fault injection.
#include <atomic>

#include "plan.h"

namespace arcs {

char* error_buffer() {
  static thread_local char buf[256] = "";
  return buf;
}

int fault_injected() {
  static const long fail_at = [] {
    const char* e = getenv("ARCS_FAIL_CALL");
    return e ? atol(e) : 0L;
  }();
  static std::atomic<long> calls{0};
  if (fail_at <= 0) return 0;
  if (++calls == fail_at) return set_error(ARCS_ERR_INJECTED, "injected failure (ARCS_FAIL_CALL)");
  return 0;
}

}  // namespace arcs

extern "C" const char* arcs_last_error(void) { return arcs::error_buffer(); }
extern "C" int arcs_version(void) { return ARCS_VERSION; }
