"""Derives, from the reference's own tests/test_sampler.cpp where it lies, the program that runs
that test against the CUDA-backed mirror of the Sampler: oracle/_ref/test_sampler_mirror.cpp
(untracked; nothing of the reference enters the repository). Two changes, both by text:
  - the include of tools/sampler.h becomes tests/cpp/sampler_shim.h, which binds `Sampler` to the
    mirror (the test's verbatim copy of the earlier implementation, `OldSampler`, stays the checker);
  - the random rows are made free of exactly equal logits (every row continuous, equal values
    nudged apart): among equal logits the reference's order is whatever its standard library's
    heap code gives, while this library orders them by token id; the number of rows this changes
    is printed by the program.
usage: make_sampler_test.py REF_DIR OUT_CPP"""
import sys

ref, out = sys.argv[1], sys.argv[2]
src = open(ref + "/tests/test_sampler.cpp").read()
inc = '#include "../tools/sampler.h"'
assert src.count(inc) == 1
src = src.replace(inc, '#include "tests/cpp/sampler_shim.h"\n#include <algorithm>\n#include <cmath>\nstatic long g_rows_made_distinct = 0, g_rows = 0;')
old = "  return l;\n}\nstatic std::vector<int> rand_recent"
assert src.count(old) == 1
new = """  {  // (derived test: no two logits of a row exactly equal)
    ++g_rows;
    if (mode != 0) {
      std::normal_distribution<float> nd2(0.0f, 3.0f);
      for (int i = 0; i < V; ++i) l[i] = nd2(g);
      ++g_rows_made_distinct;
    }
    std::vector<int> idx(V);
    for (int i = 0; i < V; ++i) idx[i] = i;
    std::sort(idx.begin(), idx.end(), [&](int a, int b) { return l[a] < l[b]; });
    bool nudged = false;
    for (int i = 1; i < V; ++i)
      if (!(l[idx[i]] > l[idx[i - 1]])) {
        l[idx[i]] = std::nextafter(l[idx[i - 1]], 1e30f);
        nudged = true;
      }
    if (nudged && mode == 0) ++g_rows_made_distinct;
  }
  return l;
}
static std::vector<int> rand_recent"""
src = src.replace(old, new)
old = '  printf("ALL OK\\n");'
assert src.count(old) == 1
src = src.replace(old, '  printf("rows with equal logits made distinct: %ld of %ld\\n", g_rows_made_distinct, g_rows);\n' + old)
open(out, "w").write(src)
