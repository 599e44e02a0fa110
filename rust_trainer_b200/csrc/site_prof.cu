// Measurement aid, compiled only with -DRT_B200_SITEPROF: the time between consecutive launch sites
// on the context's stream, as the kernels run inside a real step (warm L2, back to back), summed
// per site.  A profiler's per-kernel durations are taken with cold caches and cannot say which
// memory-bound kernel matters once its operands are still in L2.  Marks made while a stream is
// being captured become event-record nodes of the graph, so a replay stamps them on the GPU with no
// host in the loop: begin before the step is captured, replay, then end.
#include "ctx.h"
#include "rt_internal.h"
#ifdef RT_B200_SITEPROF
#include <map>
#include <string>
#include <vector>
#include <stdio.h>
#include <string.h>

namespace rt {
namespace {
struct Mark { cudaEvent_t ev; const char* file; int line; };
std::vector<Mark> g_marks;
std::vector<cudaEvent_t> g_pool;
cudaStream_t g_prof_stream = nullptr;
bool g_prof_on = false;
cudaEvent_t get_event() {
  if (!g_pool.empty()) { cudaEvent_t e = g_pool.back(); g_pool.pop_back(); return e; }
  cudaEvent_t e;
  cudaEventCreate(&e);
  return e;
}
}  // namespace
void prof_mark(const char* file, int line) {
  if (!g_prof_on) return;
  cudaEvent_t e = get_event();
  cudaEventRecord(e, g_prof_stream);
  g_marks.push_back({e, file, line});
}
}  // namespace rt

extern "C" int rt_debug_site_profile_begin(rt_ctx* c) {
  rt::g_prof_stream = c->stream;
  rt::g_prof_on = true;
  rt::prof_mark("begin", 0);
  return 0;
}
extern "C" int rt_debug_site_profile_end(char* buf, int n) {
  using namespace rt;
  g_prof_on = false;
  cudaStreamSynchronize(g_prof_stream);
  std::map<std::string, std::pair<int, double>> agg;
  double total = 0;
  for (size_t i = 1; i < g_marks.size(); ++i) {
    float ms = 0;
    cudaEventElapsedTime(&ms, g_marks[i - 1].ev, g_marks[i].ev);
    const char* f = strrchr(g_marks[i].file, '/');
    char key[128];
    snprintf(key, sizeof key, "%s:%d", f ? f + 1 : g_marks[i].file, g_marks[i].line);
    auto& a = agg[key];
    a.first += 1;
    a.second += ms;
    total += ms;
  }
  for (auto& m : g_marks) g_pool.push_back(m.ev);
  g_marks.clear();
  int off = snprintf(buf, n, "total %.3f ms\n", total);
  for (auto& kv : agg)
    if (off < n - 100) off += snprintf(buf + off, n - off, "%-28s n=%5d total=%8.3f ms avg=%8.2f us\n", kv.first.c_str(), kv.second.first, kv.second.second, kv.second.second * 1000.0 / kv.second.first);
  return off;
}
#endif
