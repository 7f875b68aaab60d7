// Host-side runtime pieces that the engine drives every step: the paged-KV block manager (free list,
// reference counts, fork with copy-on-write of the tail page), the continuous-batching scheduler (decode
// first, chunked prefill in the remaining token budget, preemption by recompute when pages run out) and
// the profiler tables.
//
// Reference counterparts: the contiguous per-layer KV buffers of common/transformer.h:2037-2079 (no paging
// exists there), the continuous-batching loop of a64fx/glm5/glm5_ep_runner.c:294-376 (finished slots are
// refilled immediately), multi-stream decode of common/m3_impl.h:870-970, and common/profiler.h:44-77,110-249
// (named timers with FLOP counts and per-op / per-type / per-component tables).
#include "common.h"
#include <string.h>
#include <algorithm>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace gbh {

// ------------------------------------------------------------------------------------------ KV block manager
struct KvSeq { std::vector<int> pages; int tokens = 0; bool live = false; };

struct KvManager {
  int num_pages, page_size;
  std::vector<int> free_list;      // stack
  std::vector<int> refcount;
  std::vector<KvSeq> seqs;
  std::vector<int> free_seq_ids;

  KvManager(int n, int ps) : num_pages(n), page_size(ps), refcount(n, 0) {
    free_list.reserve(n);
    for (int i = n - 1; i >= 0; --i) free_list.push_back(i);
  }
  int seq_new() {
    int id;
    if (!free_seq_ids.empty()) { id = free_seq_ids.back(); free_seq_ids.pop_back(); }
    else { id = (int)seqs.size(); seqs.emplace_back(); }
    seqs[id] = KvSeq(); seqs[id].live = true;
    return id;
  }
  bool valid(int s) const { return s >= 0 && s < (int)seqs.size() && seqs[s].live; }
  int pages_for(int tokens) const { return (tokens + page_size - 1) / page_size; }
  // Make room for `tokens` positions in total.  All or nothing.
  int reserve(int s, int tokens) {
    if (!valid(s)) return fail("kv: bad sequence %d", s);
    KvSeq& q = seqs[s];
    const int need = pages_for(tokens) - (int)q.pages.size();
    if (need > (int)free_list.size()) return fail("kv: out of pages (want %d, free %d)", need, (int)free_list.size());
    for (int i = 0; i < need; ++i) { const int p = free_list.back(); free_list.pop_back(); refcount[p] = 1; q.pages.push_back(p); }
    q.tokens = std::max(q.tokens, tokens);
    return 0;
  }
  void release(int s) {
    if (!valid(s)) return;
    for (int p : seqs[s].pages) if (--refcount[p] == 0) free_list.push_back(p);
    seqs[s] = KvSeq();
    free_seq_ids.push_back(s);
  }
  // New sequence sharing the first `tokens` positions of `s`.  Full pages are shared by reference count; a partly
  // filled tail page is given a fresh page and reported as a (src, dst) copy for the device to perform.
  int fork(int s, int tokens, int* copy_src, int* copy_dst) {
    *copy_src = *copy_dst = -1;
    if (!valid(s) || tokens > seqs[s].tokens) return fail("kv: cannot fork %d tokens of sequence %d", tokens, s), -1;
    const int full = tokens / page_size, tail = tokens % page_size;
    if (tail && free_list.empty()) return fail("kv: out of pages for the fork's tail page"), -1;
    const int id = seq_new();
    KvSeq& dst = seqs[id];
    const KvSeq& src = seqs[s];
    for (int i = 0; i < full; ++i) { dst.pages.push_back(src.pages[i]); ++refcount[src.pages[i]]; }
    if (tail) {
      const int p = free_list.back(); free_list.pop_back(); refcount[p] = 1;
      dst.pages.push_back(p);
      *copy_src = src.pages[full]; *copy_dst = p;
    }
    dst.tokens = tokens;
    return id;
  }
};

// ------------------------------------------------------------------------------------------ scheduler
struct Request {
  long id = 0; int prompt_len = 0; int max_new = 0;
  int computed = 0;        // prompt positions whose KV is in the cache
  int generated = 0;       // tokens produced so far
  int seq = -1;            // KV sequence (-1 = not admitted / preempted)
  long arrival = 0;
};
struct PlanItem { long req_id; int seq; int q_len; int ctx_len; int is_prefill; int emits_token; };

struct Scheduler {
  KvManager* kv; int max_running; int max_batch_tokens;
  std::deque<Request> waiting;
  std::vector<Request> running;
  std::vector<PlanItem> last_plan;
  std::vector<long> aborted;   // requests dropped because they can never be served (read and cleared by take_aborted)
  long clock = 0; long n_preempted = 0;
  int lookahead = 0;       // speculative decoding: extra positions a decode item may fill with draft tokens

  // A request whose prompt plus generation (plus look-ahead) exceeds the whole cache can never finish: refuse it up front.
  bool fits(int prompt_len, int max_new) const {
    return (long)prompt_len + std::max(max_new, 1) + lookahead <= (long)kv->num_pages * kv->page_size;
  }

  // Recompute-preemption of running[idx]: its pages go back, it restarts from position 0 at the head of the queue.
  void preempt(size_t idx, std::vector<long>& preempted_now) {
    Request v = running[idx];
    kv->release(v.seq);
    v.seq = -1; v.computed = 0; v.prompt_len += v.generated; v.max_new -= v.generated; v.generated = 0;
    preempted_now.push_back(v.id);
    waiting.push_front(v);
    running.erase(running.begin() + (long)idx);
    ++n_preempted;
  }

  // One engine step: every running sequence that finished its prompt decodes one token; what is left of the token
  // budget goes to prompt chunks, oldest request first; new requests are admitted while slots and pages allow.
  // Requests are visited oldest first, and a victim of preemption is always YOUNGER than the request that needs the page
  // (or that request itself), so no request that already owns an item of this plan is ever preempted.  A request preempted
  // in this call is not re-admitted in the same call: its sequence id could be reused inside one plan otherwise.
  int plan(std::vector<PlanItem>& out) {
    out.clear();
    int budget = max_batch_tokens;
    std::vector<long> preempted_now;
    std::sort(running.begin(), running.end(), [](const Request& a, const Request& b) { return a.arrival < b.arrival; });
    for (size_t i = 0; i < running.size();) {
      if (running[i].computed < running[i].prompt_len) { ++i; continue; }
      if (budget <= 0) break;
      const int total = running[i].prompt_len + running[i].generated + 1 + lookahead;
      bool ok = kv->reserve(running[i].seq, total) == 0;
      while (!ok && running.size() - 1 > i) {          // the youngest request behind this one gives up its pages
        preempt(running.size() - 1, preempted_now);
        ok = kv->reserve(running[i].seq, total) == 0;
      }
      if (!ok) {
        // this request is the youngest.  If older ones hold the pages it waits its turn from the queue; alone it has
        // outgrown the whole cache and can never continue.
        if (running.size() > 1) preempt(i, preempted_now);
        else { aborted.push_back(running[i].id); kv->release(running[i].seq); running.erase(running.begin() + (long)i); }
        continue;                                        // running[i] is now the next request (or the end)
      }
      const Request& rr = running[i];
      out.push_back({rr.id, rr.seq, 1, rr.prompt_len + rr.generated - 1, 0, 1});   // ctx = positions cached before this token
      budget -= 1 + lookahead; ++i;
    }
    // prompt chunks of running requests
    for (size_t i = 0; i < running.size(); ++i) {
      Request& r = running[i];
      if (budget <= 0) break;
      if (r.computed >= r.prompt_len) continue;
      const int take = std::min(budget, r.prompt_len - r.computed);
      if (kv->reserve(r.seq, r.computed + take) != 0) {
        // no page for the next chunk.  Other requests will free pages as they finish; a lone request never gets more.
        if (running.size() == 1 && out.empty()) { aborted.push_back(r.id); kv->release(r.seq); running.erase(running.begin() + (long)i); --i; }
        continue;
      }
      out.push_back({r.id, r.seq, take, r.computed, 1, (r.computed + take == r.prompt_len) ? 1 : 0});
      budget -= take;
    }
    // admissions
    while (budget > 0 && !waiting.empty() && (int)running.size() < max_running) {
      Request r = waiting.front();
      if (std::find(preempted_now.begin(), preempted_now.end(), r.id) != preempted_now.end()) break;
      if (!fits(r.prompt_len, r.max_new)) { aborted.push_back(r.id); waiting.pop_front(); continue; }
      const int take = std::min(budget, r.prompt_len);
      const int seq = kv->seq_new();
      if (kv->reserve(seq, take) != 0) {
        kv->release(seq);
        // nothing is running, so nothing will ever free a page for this chunk: shrink it to what is free, or give up
        if (running.empty() && out.empty()) {
          const int room = (int)kv->free_list.size() * kv->page_size;
          if (room <= 0) { aborted.push_back(r.id); waiting.pop_front(); continue; }
          const int seq2 = kv->seq_new();
          const int take2 = std::min(take, room);
          if (kv->reserve(seq2, take2) != 0) { kv->release(seq2); aborted.push_back(r.id); waiting.pop_front(); continue; }
          waiting.pop_front();
          r.seq = seq2; running.push_back(r);
          out.push_back({r.id, seq2, take2, 0, 1, take2 == r.prompt_len ? 1 : 0});
          budget -= take2;
          continue;
        }
        break;
      }
      waiting.pop_front();
      r.seq = seq;
      running.push_back(r);
      out.push_back({r.id, seq, take, 0, 1, take == r.prompt_len ? 1 : 0});
      budget -= take;
    }
    last_plan = out;
    return (int)out.size();
  }

  // After the step ran: advance the requests; `finished[i] != 0` marks items whose sequence hit a stop condition.
  // `advance[i]` (optional) is the number of tokens a decode item produced: 1, or more after accepted draft tokens.
  void commit(const int* finished, int n, const int* advance = nullptr) {
    for (int i = 0; i < n && i < (int)last_plan.size(); ++i) {
      const PlanItem& it = last_plan[i];
      for (size_t j = 0; j < running.size(); ++j) {
        Request& r = running[j];
        if (r.id != it.req_id) continue;
        if (it.is_prefill) { r.computed += it.q_len; if (it.emits_token) r.generated += 1; }
        else r.generated += (advance && advance[i] > 1) ? advance[i] : 1;
        const bool done = (finished && finished[i]) || r.generated >= r.max_new;
        if (done && r.computed >= r.prompt_len) { kv->release(r.seq); running.erase(running.begin() + (long)j); }
        break;
      }
    }
    last_plan.clear();
  }
};

// ------------------------------------------------------------------------------------------ profiler
struct ProfEntry { std::string name, type, component; int layer; double ns = 0, flops = 0, bytes = 0; long calls = 0; };
struct Profiler {
  std::mutex mu;
  std::map<std::string, ProfEntry> entries;
  void add(const char* name, const char* type, const char* component, int layer, double ns, double flops, double bytes) {
    std::lock_guard<std::mutex> g(mu);
    const std::string key = std::string(component) + "/" + name + "/" + std::to_string(layer);
    ProfEntry& e = entries[key];
    if (e.calls == 0) { e.name = name; e.type = type; e.component = component; e.layer = layer; }
    e.ns += ns; e.flops += flops; e.bytes += bytes; ++e.calls;
  }
  std::string summary() {
    std::lock_guard<std::mutex> g(mu);
    std::map<std::string, ProfEntry> by_op, by_type, by_comp;
    double total = 0;
    for (auto& kv : entries) {
      const ProfEntry& e = kv.second;
      for (auto* m : {&by_op, &by_type, &by_comp}) {
        const std::string& k = m == &by_op ? e.name : m == &by_type ? e.type : e.component;
        ProfEntry& a = (*m)[k];
        a.name = k; a.ns += e.ns; a.flops += e.flops; a.bytes += e.bytes; a.calls += e.calls;
      }
      total += e.ns;
    }
    std::string out;
    char line[256];
    auto table = [&](const char* title, std::map<std::string, ProfEntry>& m) {
      std::vector<ProfEntry> v;
      for (auto& kv : m) v.push_back(kv.second);
      std::sort(v.begin(), v.end(), [](const ProfEntry& a, const ProfEntry& b) { return a.ns > b.ns; });
      snprintf(line, sizeof(line), "%-28s %10s %10s %7s %10s %10s\n", title, "calls", "ms", "%", "GFLOP/s", "GB/s");
      out += line;
      for (auto& e : v) {
        snprintf(line, sizeof(line), "%-28s %10ld %10.3f %6.1f%% %10.1f %10.1f\n", e.name.c_str(), e.calls, e.ns / 1e6,
                 total > 0 ? 100.0 * e.ns / total : 0.0, e.ns > 0 ? e.flops / e.ns : 0.0, e.ns > 0 ? e.bytes / e.ns : 0.0);
        out += line;
      }
      out += "\n";
    };
    table("per op", by_op); table("per op type", by_type); table("per component", by_comp);
    snprintf(line, sizeof(line), "total %.3f ms\n", total / 1e6);
    out += line;
    return out;
  }
};
static Profiler g_prof;

}  // namespace gbh

using namespace gbh;

// ------------------------------------------------------------------------------------------ C API: KV
GBH_API void* gbh_kv_create(int num_pages, int page_size) { return new KvManager(num_pages, page_size); }
GBH_API void gbh_kv_destroy(void* h) { delete (KvManager*)h; }
GBH_API int gbh_kv_seq_new(void* h) { return ((KvManager*)h)->seq_new(); }
GBH_API int gbh_kv_seq_reserve(void* h, int seq, int tokens) { return ((KvManager*)h)->reserve(seq, tokens); }
GBH_API void gbh_kv_seq_release(void* h, int seq) { ((KvManager*)h)->release(seq); }
GBH_API int gbh_kv_seq_fork(void* h, int seq, int tokens, int* copy_src, int* copy_dst) { return ((KvManager*)h)->fork(seq, tokens, copy_src, copy_dst); }
GBH_API int gbh_kv_seq_pages(void* h, int seq, int* out, int cap) {
  auto* m = (KvManager*)h;
  if (!m->valid(seq)) return -1;
  const auto& p = m->seqs[seq].pages;
  for (int i = 0; i < (int)p.size() && i < cap; ++i) out[i] = p[i];
  return (int)p.size();
}
GBH_API int gbh_kv_num_free(void* h) { return (int)((KvManager*)h)->free_list.size(); }
GBH_API int gbh_kv_refcount(void* h, int page) { auto* m = (KvManager*)h; return (page >= 0 && page < m->num_pages) ? m->refcount[page] : -1; }

// ------------------------------------------------------------------------------------------ C API: scheduler
GBH_API void* gbh_sched_create(void* kv, int max_running, int max_batch_tokens) {
  auto* s = new Scheduler(); s->kv = (KvManager*)kv; s->max_running = max_running; s->max_batch_tokens = max_batch_tokens; return s;
}
GBH_API void gbh_sched_destroy(void* h) { delete (Scheduler*)h; }
// Returns 0, or -1 (with the error text set) when the request could never fit the cache and was not queued.
GBH_API int gbh_sched_add(void* h, long req_id, int prompt_len, int max_new) {
  auto* s = (Scheduler*)h;
  if (prompt_len <= 0) return fail("scheduler: empty prompt (request %ld)", req_id);
  if (!s->fits(prompt_len, max_new))
    return fail("scheduler: request %ld needs %d positions, the cache holds %d", req_id, prompt_len + std::max(max_new, 1) + s->lookahead,
                s->kv->num_pages * s->kv->page_size);
  Request r; r.id = req_id; r.prompt_len = prompt_len; r.max_new = max_new; r.arrival = s->clock++; s->waiting.push_back(r);
  return 0;
}
// Requests the scheduler gave up on since the last call (they can never be served: the cache is too small for them).
GBH_API int gbh_sched_take_aborted(void* h, long* out, int cap) {
  auto* s = (Scheduler*)h;
  int n = 0;
  for (long id : s->aborted) if (n < cap) out[n++] = id;
  s->aborted.clear();
  return n;
}
// Fills parallel arrays (capacity cap) and returns the number of plan items.
GBH_API int gbh_sched_plan(void* h, long* req_id, int* seq, int* q_len, int* ctx_len, int* is_prefill, int* emits, int cap) {
  auto* s = (Scheduler*)h;
  std::vector<PlanItem> items;
  s->plan(items);
  for (int i = 0; i < (int)items.size() && i < cap; ++i) {
    req_id[i] = items[i].req_id; seq[i] = items[i].seq; q_len[i] = items[i].q_len; ctx_len[i] = items[i].ctx_len;
    is_prefill[i] = items[i].is_prefill; emits[i] = items[i].emits_token;
  }
  return (int)items.size();
}
GBH_API void gbh_sched_commit(void* h, const int* finished, int n) { ((Scheduler*)h)->commit(finished, n); }
GBH_API void gbh_sched_commit_n(void* h, const int* finished, const int* advance, int n) { ((Scheduler*)h)->commit(finished, n, advance); }
GBH_API void gbh_sched_set_lookahead(void* h, int extra) { ((Scheduler*)h)->lookahead = extra < 0 ? 0 : extra; }
GBH_API int gbh_sched_num_waiting(void* h) { return (int)((Scheduler*)h)->waiting.size(); }
GBH_API int gbh_sched_num_running(void* h) { return (int)((Scheduler*)h)->running.size(); }
GBH_API long gbh_sched_num_preempted(void* h) { return ((Scheduler*)h)->n_preempted; }

// ------------------------------------------------------------------------------------------ C API: profiler
GBH_API void gbh_prof_add(const char* name, const char* type, const char* component, int layer, double ns, double flops, double bytes) {
  g_prof.add(name, type, component, layer, ns, flops, bytes);
}
GBH_API void gbh_prof_reset() { std::lock_guard<std::mutex> g(g_prof.mu); g_prof.entries.clear(); }
GBH_API long gbh_prof_summary(char* out, long cap) {
  const std::string s = g_prof.summary();
  const long n = std::min<long>((long)s.size(), cap - 1);
  if (n > 0) memcpy(out, s.data(), (size_t)n);
  if (cap > 0) out[std::max<long>(n, 0)] = 0;
  return (long)s.size();
}
