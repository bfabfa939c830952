// The host runtime of the engine: page pools and block tables, request slots, the scheduler and the
// packing of a step's metadata.  Plain C++17, no device code and no CUDA calls; the Python classes in
// flint_b200/cache and flint_b200/engine are thin faces of these objects (ctypes, C linkage).
//
// The reference keeps the same pieces native: the paged pool with a LIFO free list and one table per
// sequence slot (crates/thuban_model/src/pool.rs:11-118), the per-row metadata of a step
// (crates/thuban_model/src/rows.rs:7-30) and the engine that admits, cuts prompts into portions, decodes and
// frees (crates/thuban_generate/src/engine.rs, resolver.rs).  Unlike the reference, a group of layers with a
// sliding window gives pages back as soon as no later query can reach them, and when pages run out the
// youngest running request is preempted and recomputed later.
//
// Every function returns 0 (or a count) on success and a negative code on failure; the message of the last
// failure of the calling thread is read with flint_rt_last_error().
#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <string>
#include <vector>

namespace {

thread_local char g_error[512];

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

constexpr int NO_PAGE = -1;
// failure codes: the Python face maps them to its exception classes
constexpr int E_CACHE = -1;      // pages, slots, context limit
constexpr int E_MODEL = -2;      // a malformed step
constexpr int E_CHECK = -3;      // a broken invariant (tests)

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ------------------------------------------------------------------------------------------------ pages
// Pages of one layer group: a pool of page numbers with a LIFO free list (a page just freed is the next one
// handed out, which keeps reuse frequent and easy to test) and one table per request slot.  Entries of a
// table before first_live have been given back (window) and read NO_PAGE.
struct Group {
  int n_pages, page_size, window, max_pages;
  std::vector<int> free_list;
  std::vector<char> held;
  std::vector<int> served;          // how many times each page was handed out
  long long total_allocations = 0;
  struct Table {
    std::vector<int> pages;
    int first_live = 0;
  };
  std::vector<Table> tables;
  std::vector<char> dirty;          // slots whose table changed since the last sync
  int* host_table = nullptr;        // [slots, max_pages] mirror that is copied to the device, or null

  Group(int n, int page, int win, int slots, int max_pages_per_request, int* mirror)
      : n_pages(n), page_size(page), window(win), max_pages(max_pages_per_request), held(n, 0), served(n, 0),
        tables(slots), dirty(slots, 0), host_table(mirror) {
    free_list.reserve(n);
    for (int p = n - 1; p >= 0; --p) free_list.push_back(p);
  }
  int free_pages() const { return (int)free_list.size(); }
  int used_pages() const { return n_pages - (int)free_list.size(); }
  // the first position a query at pos can still see
  int first_visible(int pos) const { return window ? std::max(0, pos + 1 - window) : 0; }

  int take() {
    if (free_list.empty()) return fail(E_CACHE, "page pool exhausted");
    const int p = free_list.back();
    free_list.pop_back();
    if (held[p]) return fail(E_CHECK, "page %d handed out twice", p);
    held[p] = 1;
    ++total_allocations;
    ++served[p];
    return p;
  }
  int give_back(int page) {
    if (page < 0 || page >= n_pages || !held[page]) return fail(E_CACHE, "page %d freed twice or never allocated", page);
    held[page] = 0;
    free_list.push_back(page);
    return 0;
  }
  void touch(int slot) {
    dirty[slot] = 1;
    if (host_table) {
      int* row = host_table + (size_t)slot * max_pages;
      const Table& t = tables[slot];
      const int n = std::min((int)t.pages.size(), max_pages);
      for (int i = 0; i < n; ++i) row[i] = t.pages[i];
      for (int i = n; i < max_pages; ++i) row[i] = NO_PAGE;
    }
  }
  // new pages to run positions [start, end) of this request
  int pages_needed(int slot, int start, int end) const {
    const Table& t = tables[slot];
    const int want_hi = ceil_div(end, page_size);
    const int lo = std::max((int)t.pages.size(), first_visible(start) / page_size);
    return std::max(0, want_hi - lo);
  }
  // make pages exist for positions [first_visible(start), end)
  int ensure(int slot, int start, int end) {
    Table& t = tables[slot];
    const int want_hi = ceil_div(end, page_size);
    if (want_hi > max_pages) return fail(E_CACHE, "context limit %d reached", max_pages * page_size);
    const int need = pages_needed(slot, start, end);
    if (need > free_pages()) return fail(E_CACHE, "page pool exhausted: %d pages requested, %d free", need, free_pages());
    const int first = first_visible(start) / page_size;
    bool changed = false;
    while ((int)t.pages.size() < want_hi) {
      const int i = (int)t.pages.size();
      if (i < first) {
        t.pages.push_back(NO_PAGE);      // never needed: behind the window from the start
        t.first_live = std::max(t.first_live, i + 1);
      } else {
        const int p = take();
        if (p < 0) return p;
        t.pages.push_back(p);
      }
      changed = true;
    }
    if (changed) touch(slot);
    return 0;
  }
  // give back pages that no query at next_pos or later can see
  int release_behind(int slot, int next_pos) {
    if (!window) return 0;
    Table& t = tables[slot];
    const int dead_hi = std::min(first_visible(next_pos) / page_size, (int)t.pages.size());
    int n = 0;
    for (int i = t.first_live; i < dead_hi; ++i)
      if (t.pages[i] != NO_PAGE) {
        if (int rc = give_back(t.pages[i])) return rc;
        t.pages[i] = NO_PAGE;
        ++n;
      }
    if (dead_hi > t.first_live) {
      t.first_live = dead_hi;
      touch(slot);
    }
    return n;
  }
  int release_all(int slot) {
    Table& t = tables[slot];
    int n = 0;
    for (int p : t.pages)
      if (p != NO_PAGE) {
        if (int rc = give_back(p)) return rc;
        ++n;
      }
    t.pages.clear();
    t.first_live = 0;
    touch(slot);
    return n;
  }
  // drop pages above keep_tokens positions (crates/thuban_model/src/pool.rs:73-79)
  int truncate(int slot, int keep_tokens) {
    Table& t = tables[slot];
    const int keep = std::min(ceil_div(keep_tokens, page_size), (int)t.pages.size());
    for (int i = keep; i < (int)t.pages.size(); ++i)
      if (t.pages[i] != NO_PAGE)
        if (int rc = give_back(t.pages[i])) return rc;
    t.pages.resize(keep);
    t.first_live = std::min(t.first_live, keep);
    touch(slot);
    return 0;
  }
  // invariants: every page is either free exactly once or held (the pool alone), and, with the tables, held
  // by exactly one request
  int check(bool with_tables = true) const {
    std::vector<char> is_free(n_pages, 0);
    for (int p : free_list) {
      if (p < 0 || p >= n_pages || is_free[p]) return fail(E_CHECK, "a page is on the free list twice");
      is_free[p] = 1;
    }
    for (int p = 0; p < n_pages; ++p)
      if ((held[p] != 0) == (is_free[p] != 0)) return fail(E_CHECK, "page %d both held and free (or neither)", p);
    if (!with_tables) return 0;
    std::vector<char> seen(n_pages, 0);
    int n_seen = 0;
    for (const Table& t : tables)
      for (int p : t.pages)
        if (p != NO_PAGE) {
          if (p < 0 || p >= n_pages || seen[p]) return fail(E_CHECK, "page %d held by two requests", p);
          seen[p] = 1;
          ++n_seen;
        }
    if (n_seen != used_pages()) return fail(E_CHECK, "a page is lost (held by no request, not free)");
    return 0;
  }
};

// ------------------------------------------------------------------------------------------------ slots
// Slots and pages of all requests of one model: the groups (owned by their Python faces) plus the free list
// of request slots.
struct Cache {
  int page_size, max_slots, max_context;
  std::vector<Group*> groups;
  std::vector<int> free_slots;
  std::vector<char> live;
  Cache(int page, int slots, int ctx) : page_size(page), max_slots(slots), max_context(ctx), live(slots, 0) {
    for (int s = slots - 1; s >= 0; --s) free_slots.push_back(s);
  }
  int admit() {
    if (free_slots.empty()) return fail(E_CACHE, "no free request slot");
    const int s = free_slots.back();
    free_slots.pop_back();
    live[s] = 1;
    return s;
  }
  int release(int slot) {
    if (slot < 0 || slot >= max_slots || !live[slot]) return fail(E_CACHE, "slot %d released twice or never admitted", slot);
    for (Group* g : groups)
      if (int rc = g->release_all(slot); rc < 0) return rc;
    live[slot] = 0;
    free_slots.push_back(slot);
    return 0;
  }
  int pages_needed(int slot, int start, int end) const {
    int n = 0;
    for (const Group* g : groups) n = std::max(n, g->pages_needed(slot, start, end));
    return n;
  }
  int free_pages() const {
    int n = 1 << 30;
    for (const Group* g : groups) n = std::min(n, g->free_pages());
    return n;
  }
  bool can_run(int slot, int start, int end) const {
    if (end > max_context) return false;
    for (const Group* g : groups)
      if (g->pages_needed(slot, start, end) > g->free_pages()) return false;
    return true;
  }
  int ensure(int slot, int start, int end) {
    if (slot < 0 || slot >= max_slots || !live[slot]) return fail(E_CACHE, "slot %d is not admitted", slot);
    if (end > max_context) return fail(E_CACHE, "context limit %d reached", max_context);
    if (!can_run(slot, start, end))
      return fail(E_CACHE, "page pool exhausted: slot %d needs %d pages, %d free", slot, pages_needed(slot, start, end),
                  free_pages());
    for (Group* g : groups)
      if (int rc = g->ensure(slot, start, end); rc < 0) return rc;
    return 0;
  }
  int advance(int slot, int next_pos) {
    for (Group* g : groups)
      if (int rc = g->release_behind(slot, next_pos); rc < 0) return rc;
    return 0;
  }
  bool windowed() const {
    for (const Group* g : groups)
      if (g->window) return true;
    return false;
  }
  int check() const {
    for (const Group* g : groups)
      if (int rc = g->check()) return rc;
    std::vector<char> is_free(max_slots, 0);
    for (int s : free_slots) {
      if (s < 0 || s >= max_slots || is_free[s]) return fail(E_CHECK, "a slot is on the free list twice");
      if (live[s]) return fail(E_CHECK, "slot %d both free and live", s);
      is_free[s] = 1;
    }
    int n_live = 0;
    for (char l : live) n_live += l != 0;
    if ((int)free_slots.size() + n_live != max_slots) return fail(E_CHECK, "a slot is lost");
    return 0;
  }
};

// ------------------------------------------------------------------------------------------------ scheduler
// Each step: 1. decoding requests, 2. running requests with prompt (or recomputation) left, each oldest
// first, 3. waiting requests admitted first come first served while a slot, budget and pages last.  A portion
// is at most prefill_chunk tokens and the step at most max_step_tokens.  When pages run out for a running
// request, running requests that arrived after it are preempted, the last one first (pages and slot given
// back, recomputed later from the head of the queue); an older request never loses to a younger one, and a
// request that cannot fit alone fails alone.
enum State { WAITING = 0, RUNNING = 1, FINISHED = 2, FAILED = 3 };
constexpr int UNREAD = -1;          // a sampled token whose value the host has not read yet
enum Reason { R_NONE = 0, R_STOP = 1, R_LENGTH = 2, R_CONTEXT = 3, R_ABORT = 4, R_ERROR = 5 };

struct Request {
  int n_prompt = 0, n_generated = 0, max_tokens = 0, arrival = 0;
  int n_cached = 0, slot = -1, state = WAITING, reason = R_NONE;
  int preemptions = 0, prefill_tokens = 0, decode_tokens = 0;
  int n_unread = 0;       // the last n_unread generated tokens were committed before their values were read
  std::vector<int> stop;
  std::string error;
  int n_tokens() const { return n_prompt + n_generated; }
  int remaining() const { return n_tokens() - n_cached; }
};

struct Portion {
  int req, start, n_tokens, wants_logits;
};

struct Scheduler {
  Cache* cache;
  int max_step_tokens, prefill_chunk, max_context, page_size, total_pages;
  std::vector<Request> reqs;
  std::deque<int> waiting;
  std::vector<int> running;
  int preemptions = 0, steps = 0;
  std::vector<int> touched;        // requests whose state changed outside a portion (for the caller's mirrors)
  std::vector<int> free_handles;   // records of ended requests that the caller has let go of

  void fail_request(int r, const std::string& msg) {
    touched.push_back(r);
    reqs[r].state = FAILED;
    reqs[r].error = msg;
    reqs[r].reason = R_ERROR;
  }
  bool is_running(int r) const { return std::find(running.begin(), running.end(), r) != running.end(); }
  void drop_running(int r) { running.erase(std::remove(running.begin(), running.end(), r), running.end()); }

  int add(int n_prompt, int max_tokens, int arrival, const int* stop, int n_stop) {
    Request q;
    q.n_prompt = n_prompt;
    q.max_tokens = max_tokens;
    q.arrival = arrival;
    q.stop.assign(stop, stop + n_stop);
    int r;
    if (!free_handles.empty()) {          // the record of a request that the caller has forgotten is used again
      r = free_handles.back();
      free_handles.pop_back();
      reqs[r] = q;
    } else {
      reqs.push_back(q);
      r = (int)reqs.size() - 1;
    }
    char buf[160];
    if (n_prompt <= 0) {
      fail_request(r, "empty prompt");
    } else if (n_prompt + 1 > max_context) {
      snprintf(buf, sizeof(buf), "prompt of %d tokens does not fit the context limit %d", n_prompt, max_context);
      fail_request(r, buf);
    } else {
      waiting.push_back(r);
    }
    return r;
  }
  // give back the pages and the slot of a running request; it will be recomputed
  int preempt(int victim) {
    if (reqs[victim].n_unread) return fail(E_CHECK, "a request with unread tokens cannot be recomputed");
    drop_running(victim);
    if (int rc = cache->release(reqs[victim].slot)) return rc;
    Request& v = reqs[victim];
    v.slot = -1;
    v.n_cached = 0;
    v.state = WAITING;
    ++v.preemptions;
    ++preemptions;
    touched.push_back(victim);
    waiting.push_front(victim);
    return 0;
  }
  // largest m <= n such that pages exist for positions [n_cached, n_cached + m)
  int fits_portion(int r, int n) const {
    const Request& q = reqs[r];
    while (n > 0 && !cache->can_run(q.slot, q.n_cached, q.n_cached + n))
      n = n > page_size ? (n - 1) / page_size * page_size : n - 1;
    return n;
  }
  // pages ran out for r: preempt running requests that arrived after it, the last one first, until at least
  // one token of r fits.  Returns the budget given back by voided portions (or a negative code).
  int make_room(int r, std::vector<Portion>& portions) {
    int refund = 0;
    while (is_running(r) && !cache->can_run(reqs[r].slot, reqs[r].n_cached, reqs[r].n_cached + 1)) {
      int victim = -1;
      for (int o : running)
        if (reqs[o].arrival > reqs[r].arrival && (victim < 0 || reqs[o].arrival > reqs[victim].arrival)) victim = o;
      if (victim < 0) {
        if (running.size() == 1) {
          drop_running(r);
          if (int rc = cache->release(reqs[r].slot)) return rc;
          reqs[r].slot = -1;
          char buf[160];
          snprintf(buf, sizeof(buf), "request of %d tokens needs more pages than the pool has", reqs[r].n_tokens());
          fail_request(r, buf);
          break;
        }
        victim = r;       // the others are older and go first
      }
      for (size_t i = 0; i < portions.size();)
        if (portions[i].req == victim) {
          refund += portions[i].n_tokens;
          portions.erase(portions.begin() + i);
        } else {
          ++i;
        }
      if (int rc = preempt(victim)) return rc;
    }
    return refund;
  }
  bool planned(const std::vector<Portion>& portions, int r) const {
    for (const Portion& p : portions)
      if (p.req == r) return true;
    return false;
  }
  int plan(std::vector<Portion>& portions) {
    int budget = max_step_tokens;
    portions.clear();
    for (int pass = 0; pass < 2; ++pass) {
      const bool decoding = pass == 0;
      std::vector<int> order(running);
      std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return reqs[a].arrival < reqs[b].arrival; });
      for (int r : order) {
        if (!is_running(r) || planned(portions, r) || budget <= 0 || reqs[r].remaining() < 1) continue;
        if (decoding != (reqs[r].remaining() == 1)) continue;
        int n = fits_portion(r, std::min({reqs[r].remaining(), prefill_chunk, budget}));
        if (n == 0) {
          const int refund = make_room(r, portions);
          if (refund < 0) return refund;
          budget += refund;
          if (!is_running(r)) continue;
          n = fits_portion(r, std::min({reqs[r].remaining(), prefill_chunk, budget}));
          if (n == 0) continue;
        }
        Request& q = reqs[r];
        if (int rc = cache->ensure(q.slot, q.n_cached, q.n_cached + n)) return rc;
        portions.push_back({r, q.n_cached, n, n == q.remaining() ? 1 : 0});
        budget -= n;
      }
    }
    // waiting requests, first come first served; admission never preempts
    while (!waiting.empty() && budget > 0 && !cache->free_slots.empty()) {
      const int r = waiting.front();
      Request& q = reqs[r];
      const int need_pages = ceil_div(q.n_tokens(), page_size);
      if (q.n_tokens() + 1 > max_context || (need_pages > total_pages && !cache->windowed())) {
        waiting.pop_front();
        char buf[200];
        snprintf(buf, sizeof(buf), "request of %d tokens can never fit (%d pages of %d, context limit %d)", q.n_tokens(),
                 total_pages, page_size, max_context);
        fail_request(r, buf);
        continue;
      }
      const int slot = cache->admit();
      if (slot < 0) return slot;
      q.slot = slot;
      const int n = fits_portion(r, std::min({q.remaining(), prefill_chunk, budget}));
      if (n == 0) {
        if (int rc = cache->release(slot)) return rc;
        q.slot = -1;
        break;                            // no pages now; it keeps its place at the head
      }
      waiting.pop_front();
      q.state = RUNNING;
      running.push_back(r);
      if (int rc = cache->ensure(slot, q.n_cached, q.n_cached + n)) return rc;
      portions.push_back({r, q.n_cached, n, n == q.remaining() ? 1 : 0});
      budget -= n;
    }
    ++steps;
    return 0;
  }
  int finish(int r, int reason) {
    Request& q = reqs[r];
    touched.push_back(r);
    q.state = FINISHED;
    q.reason = reason;
    drop_running(r);
    if (q.slot >= 0) {
      if (int rc = cache->release(q.slot)) return rc;
      q.slot = -1;
    }
    return 0;
  }
  // sampled: one token per portion that wanted logits, in order.  emitted: (request, token) pairs.
  int commit(const Portion* portions, int n_portions, const int* sampled, int n_sampled, std::vector<int>& emitted) {
    emitted.clear();
    int next = 0;
    for (int i = 0; i < n_portions; ++i) {
      const Portion& p = portions[i];
      Request& q = reqs[p.req];
      if (p.n_tokens == 1 && p.start >= q.n_prompt) ++q.decode_tokens;
      else q.prefill_tokens += p.n_tokens;
      q.n_cached = p.start + p.n_tokens;
      if (int rc = cache->advance(q.slot, q.n_cached)) return rc;
      if (!p.wants_logits) continue;
      if (next >= n_sampled) return fail(E_MODEL, "fewer sampled tokens than portions that wanted logits");
      const int token = sampled[next++];
      if (token == UNREAD) {
        ++q.n_unread;                   // its value, and whether it stops the request, come with resolve()
      } else if (q.n_unread) {
        return fail(E_MODEL, "a token was committed while earlier ones of its request are unread");
      } else if (std::find(q.stop.begin(), q.stop.end(), token) != q.stop.end()) {
        if (int rc = finish(p.req, R_STOP)) return rc;
        continue;
      }
      ++q.n_generated;
      emitted.push_back(p.req);
      emitted.push_back(token);
      if (q.n_generated >= q.max_tokens) {
        if (int rc = finish(p.req, R_LENGTH)) return rc;
      } else if (q.n_tokens() + 1 > max_context) {
        if (int rc = finish(p.req, R_CONTEXT)) return rc;
      }
    }
    return 0;
  }
  // The value of the oldest unread token of r.  0: it is the request's next token; 1: it is a stop token, the
  // request ends before it and what was run after it is void; 2: nothing of r is unread any more (the request
  // ended at an earlier token or was aborted), the value is dropped.
  int resolve(int r, int token) {
    Request& q = reqs[r];
    if (q.n_unread == 0) return 2;
    if (std::find(q.stop.begin(), q.stop.end(), token) == q.stop.end()) {
      --q.n_unread;
      return 0;
    }
    q.n_generated -= q.n_unread;
    q.n_unread = 0;
    if (q.state == RUNNING) {
      if (int rc = finish(r, R_STOP)) return rc;
    } else {
      q.reason = R_STOP;              // it had reached its length with this very token
      touched.push_back(r);
    }
    return 1;
  }
  // nothing waits, every running request has exactly its next token left to run, and pages for one more token
  // of each are free: the next step can be planned before the last one's tokens are read
  bool steady() const {
    if (!waiting.empty() || running.empty()) return false;
    for (int r : running)
      if (reqs[r].remaining() != 1) return false;
    return cache->free_pages() >= (int)running.size();
  }
  // the caller keeps no reference to an ended request any more: its record may serve a new one
  int forget(int r) {
    if (r < 0 || r >= (int)reqs.size()) return fail(E_MODEL, "no such request %d", r);
    if (reqs[r].state != FINISHED && reqs[r].state != FAILED) return fail(E_MODEL, "request %d has not ended", r);
    touched.erase(std::remove(touched.begin(), touched.end(), r), touched.end());
    free_handles.push_back(r);
    return 0;
  }
  int abort(int r) {
    waiting.erase(std::remove(waiting.begin(), waiting.end(), r), waiting.end());
    reqs[r].n_generated -= reqs[r].n_unread;
    reqs[r].n_unread = 0;
    return finish(r, R_ABORT);
  }
};

}  // namespace

// ================================================================================================ C face
extern "C" {

const char* flint_rt_last_error() { return g_error; }

// ---- one layer group's pages
void* flint_rt_group_create(int n_pages, int page_size, int window, int max_slots, int max_pages_per_request,
                            int* host_table) {
  if (n_pages <= 0) {
    fail(E_CACHE, "a page pool needs at least one page");
    return nullptr;
  }
  return new Group(n_pages, page_size, window, max_slots, max_pages_per_request, host_table);
}
void flint_rt_group_destroy(void* g) { delete (Group*)g; }
int flint_rt_group_take(void* g) { return ((Group*)g)->take(); }
int flint_rt_group_give_back(void* g, int page) { return ((Group*)g)->give_back(page); }
int flint_rt_group_free_pages(void* g) { return ((Group*)g)->free_pages(); }
long long flint_rt_group_total_allocations(void* g) { return ((Group*)g)->total_allocations; }
void flint_rt_group_served(void* g, int* out) {
  const Group* p = (Group*)g;
  std::copy(p->served.begin(), p->served.end(), out);
}
int flint_rt_group_pages_needed(void* g, int slot, int start, int end) { return ((Group*)g)->pages_needed(slot, start, end); }
int flint_rt_group_ensure(void* g, int slot, int start, int end) { return ((Group*)g)->ensure(slot, start, end); }
int flint_rt_group_release_behind(void* g, int slot, int next_pos) { return ((Group*)g)->release_behind(slot, next_pos); }
int flint_rt_group_release_all(void* g, int slot) { return ((Group*)g)->release_all(slot); }
int flint_rt_group_truncate(void* g, int slot, int keep_tokens) { return ((Group*)g)->truncate(slot, keep_tokens); }
int flint_rt_group_check(void* g, int with_tables) { return ((Group*)g)->check(with_tables != 0); }
// the table of a slot: returns its length, copies up to cap entries
int flint_rt_group_table(void* g, int slot, int* out, int cap) {
  const Group::Table& t = ((Group*)g)->tables[slot];
  const int n = (int)t.pages.size();
  for (int i = 0; i < n && i < cap; ++i) out[i] = t.pages[i];
  return n;
}
int flint_rt_group_first_live(void* g, int slot) { return ((Group*)g)->tables[slot].first_live; }
// the range of slots whose tables changed since the last call (lo >= hi: none); clears the marks
void flint_rt_group_take_dirty(void* g, int* lo, int* hi) {
  Group* p = (Group*)g;
  int a = (int)p->dirty.size(), b = 0;
  for (int s = 0; s < (int)p->dirty.size(); ++s)
    if (p->dirty[s]) {
      a = std::min(a, s);
      b = s + 1;
      p->dirty[s] = 0;
    }
  *lo = a;
  *hi = b;
}

// ---- slots and pages of one model
void* flint_rt_cache_create(int page_size, int max_slots, int max_context) { return new Cache(page_size, max_slots, max_context); }
void flint_rt_cache_destroy(void* c) { delete (Cache*)c; }
void flint_rt_cache_add_group(void* c, void* g) { ((Cache*)c)->groups.push_back((Group*)g); }
int flint_rt_cache_admit(void* c) { return ((Cache*)c)->admit(); }
int flint_rt_cache_release(void* c, int slot) { return ((Cache*)c)->release(slot); }
int flint_rt_cache_free_slots(void* c) { return (int)((Cache*)c)->free_slots.size(); }
int flint_rt_cache_is_live(void* c, int slot) {
  const Cache* p = (Cache*)c;
  return slot >= 0 && slot < p->max_slots && p->live[slot];
}
int flint_rt_cache_pages_needed(void* c, int slot, int start, int end) { return ((Cache*)c)->pages_needed(slot, start, end); }
int flint_rt_cache_free_pages(void* c) { return ((Cache*)c)->free_pages(); }
int flint_rt_cache_can_run(void* c, int slot, int start, int end) { return ((Cache*)c)->can_run(slot, start, end) ? 1 : 0; }
int flint_rt_cache_ensure(void* c, int slot, int start, int end) { return ((Cache*)c)->ensure(slot, start, end); }
int flint_rt_cache_advance(void* c, int slot, int next_pos) { return ((Cache*)c)->advance(slot, next_pos); }
int flint_rt_cache_check(void* c) { return ((Cache*)c)->check(); }

// ---- scheduler
void* flint_rt_sched_create(void* cache, int max_step_tokens, int prefill_chunk, int max_context, int page_size,
                            int total_pages) {
  Scheduler* s = new Scheduler();
  s->cache = (Cache*)cache;
  s->max_step_tokens = max_step_tokens;
  s->prefill_chunk = prefill_chunk;
  s->max_context = max_context;
  s->page_size = page_size;
  s->total_pages = total_pages;
  return s;
}
void flint_rt_sched_destroy(void* s) { delete (Scheduler*)s; }
// returns the handle of the new request (it may have failed at once: read its state)
int flint_rt_sched_add(void* s, int n_prompt, int max_tokens, int arrival, const int* stop, int n_stop) {
  return ((Scheduler*)s)->add(n_prompt, max_tokens, arrival, stop, n_stop);
}
void flint_rt_sched_set_stop(void* s, int r, const int* stop, int n_stop) {
  ((Scheduler*)s)->reqs[r].stop.assign(stop, stop + n_stop);
}
// out: up to cap portions of four ints (request, start, tokens, wants logits); returns their number
int flint_rt_sched_plan(void* s, int* out, int cap) {
  std::vector<Portion> portions;
  if (int rc = ((Scheduler*)s)->plan(portions)) return rc;
  if ((int)portions.size() > cap) return fail(E_MODEL, "more portions than the caller has room for");
  for (size_t i = 0; i < portions.size(); ++i) {
    out[4 * i] = portions[i].req;
    out[4 * i + 1] = portions[i].start;
    out[4 * i + 2] = portions[i].n_tokens;
    out[4 * i + 3] = portions[i].wants_logits;
  }
  return (int)portions.size();
}
// portions as given by plan; emitted: up to cap pairs (request, token); returns the number of pairs
int flint_rt_sched_commit(void* s, const int* portions, int n_portions, const int* sampled, int n_sampled, int* emitted,
                          int cap) {
  std::vector<Portion> ps(n_portions);
  for (int i = 0; i < n_portions; ++i) ps[i] = {portions[4 * i], portions[4 * i + 1], portions[4 * i + 2], portions[4 * i + 3]};
  std::vector<int> out;
  if (int rc = ((Scheduler*)s)->commit(ps.data(), n_portions, sampled, n_sampled, out)) return rc;
  if ((int)out.size() > 2 * cap) return fail(E_MODEL, "more emitted tokens than the caller has room for");
  std::copy(out.begin(), out.end(), emitted);
  return (int)out.size() / 2;
}
int flint_rt_sched_abort(void* s, int r) { return ((Scheduler*)s)->abort(r); }
int flint_rt_sched_forget(void* s, int r) { return ((Scheduler*)s)->forget(r); }
// how many request records exist (in use or waiting to be used again)
int flint_rt_sched_records(void* s) { return (int)((Scheduler*)s)->reqs.size(); }
int flint_rt_sched_resolve(void* s, int r, int token) { return ((Scheduler*)s)->resolve(r, token); }
int flint_rt_sched_steady(void* s) { return ((Scheduler*)s)->steady() ? 1 : 0; }
int flint_rt_sched_has_work(void* s) {
  const Scheduler* p = (Scheduler*)s;
  return !p->waiting.empty() || !p->running.empty();
}
// state of a request: n_generated, n_cached, slot, state, reason, preemptions, prefill_tokens, decode_tokens
void flint_rt_sched_request(void* s, int r, int* out) {
  const Request& q = ((Scheduler*)s)->reqs[r];
  const int v[8] = {q.n_generated, q.n_cached, q.slot, q.state, q.reason, q.preemptions, q.prefill_tokens, q.decode_tokens};
  std::copy(v, v + 8, out);
}
const char* flint_rt_sched_request_error(void* s, int r) { return ((Scheduler*)s)->reqs[r].error.c_str(); }
// which: 0 = waiting (in queue order), 1 = running (in admission order); returns the count
int flint_rt_sched_list(void* s, int which, int* out, int cap) {
  const Scheduler* p = (Scheduler*)s;
  int n = 0;
  if (which == 0) {
    for (int r : p->waiting) {
      if (n < cap) out[n] = r;
      ++n;
    }
  } else {
    for (int r : p->running) {
      if (n < cap) out[n] = r;
      ++n;
    }
  }
  return n;
}
// requests whose state changed since the last call other than by being given a portion; returns their number
int flint_rt_sched_take_touched(void* s, int* out, int cap) {
  Scheduler* p = (Scheduler*)s;
  const int n = (int)p->touched.size();
  for (int i = 0; i < n && i < cap; ++i) out[i] = p->touched[i];
  p->touched.clear();
  return n;
}
void flint_rt_sched_counters(void* s, int* preemptions, int* steps) {
  *preemptions = ((Scheduler*)s)->preemptions;
  *steps = ((Scheduler*)s)->steps;
}

// ---- packing of a step
// Entries: slot, start position, number of tokens, number of wanted places of each; their tokens and wanted
// places laid end to end.  Fills the host buffer (regions of `m` ints, but the tiles' of 4 * max_tiles: token
// ids, positions, slots, wanted rows, rows outside any tile, tiles of four ints, and for each row the place
// in the sampler's last output that holds its token, or -1) and
// meta = {tokens, wanted rows, tiles, other rows, largest position + 1, rows fed from the sampler's output};
// entry_start gets the first row of each entry.  Portions of at least tile_min rows are cut into tiles of up
// to tile_rows consecutive rows.  feed (may be null): for each entry -1, or the place in the sampler's last
// output whose token is the entry's first one (the host does not know its value yet).
int flint_rt_pack_step(int n_entries, const int* slots, const int* start_pos, const int* n_tokens, const int* n_want,
                       const int* tokens, const int* want, const int* feed, int vocab_size, int max_positions, int m,
                       int max_tiles, int tile_rows, int tile_min, int max_slots_seen, int* host, int* entry_start,
                       int* meta) {
  long long total = 0;
  for (int e = 0; e < n_entries; ++e) total += n_tokens[e];
  if (total == 0) return fail(E_MODEL, "a step needs at least one token");
  if (total > m) return fail(E_MODEL, "step of %lld tokens exceeds the limit of %d", total, m);
  std::vector<char> seen(std::max(max_slots_seen, 1), 0);
  int* ids = host;
  int* pos = host + m;
  int* slot = host + 2 * (size_t)m;
  int* want_rows = host + 3 * (size_t)m;
  int* others = host + 4 * (size_t)m;
  int* tiles = host + 5 * (size_t)m;
  int* fed = tiles + 4 * (size_t)max_tiles;
  int T = 0, R = 0, n_tiles = 0, n_others = 0, max_kv = 0, tok_off = 0, want_off = 0, n_fed = 0;
  for (int e = 0; e < n_entries; ++e) {
    const int s = slots[e], n = n_tokens[e], p0 = start_pos[e];
    if (s >= 0 && s < (int)seen.size()) {
      if (seen[s]) return fail(E_MODEL, "request slot %d appears twice in one step", s);
      seen[s] = 1;
    } else {
      for (int o = 0; o < e; ++o)
        if (slots[o] == s) return fail(E_MODEL, "request slot %d appears twice in one step", s);
    }
    if (n == 0) return fail(E_MODEL, "an entry needs at least one token");
    if (p0 < 0 || p0 + n > max_positions)
      return fail(E_MODEL, "positions %d..%d exceed the model's %d positions", p0, p0 + n - 1, max_positions);
    const int base = T;
    entry_start[e] = base;
    const int from = feed ? feed[e] : -1;
    if (from >= m) return fail(E_MODEL, "an entry's token is fed from place %d of at most %d", from, m);
    for (int i = 0; i < n; ++i) {
      int t = tokens[tok_off + i];
      fed[T] = -1;
      if (i == 0 && from >= 0) {
        fed[T] = from;
        ++n_fed;
        t = 0;                          // replaced on the device before the step runs
      }
      if (t < 0 || t >= vocab_size) return fail(E_MODEL, "token id %d is outside the vocabulary of %d", t, vocab_size);
      ids[T] = t;
      pos[T] = p0 + i;
      slot[T] = s;
      ++T;
    }
    tok_off += n;
    for (int i = 0; i < n_want[e]; ++i) {
      const int w = want[want_off + i];
      if (w < 0 || w >= n) return fail(E_MODEL, "wanted place %d is outside the entry's %d tokens", w, n);
      want_rows[R++] = base + w;
    }
    want_off += n_want[e];
    if (n >= tile_min) {
      for (int r = 0; r < n; r += tile_rows) {
        if (n_tiles >= max_tiles) return fail(E_MODEL, "more attention tiles than the staging buffer holds");
        int* t = tiles + 4 * (size_t)n_tiles++;
        t[0] = base + r;
        t[1] = std::min(tile_rows, n - r);
        t[2] = s;
        t[3] = p0 + r;
      }
    } else {
      for (int i = 0; i < n; ++i) others[n_others++] = base + i;
    }
    max_kv = std::max(max_kv, p0 + n);
  }
  // tiles in the order of their last position: a kernel whose work grows with the keys a tile sees starts
  // from the far end and fills in with the short ones
  {
    struct Tile { int v[4]; };
    Tile* t = reinterpret_cast<Tile*>(tiles);
    std::stable_sort(t, t + n_tiles, [](const Tile& a, const Tile& b) { return a.v[3] + a.v[1] < b.v[3] + b.v[1]; });
  }
  meta[0] = T;
  meta[1] = R;
  meta[2] = n_tiles;
  meta[3] = n_others;
  meta[4] = max_kv;
  meta[5] = n_fed;
  return 0;
}

}  // extern "C"
