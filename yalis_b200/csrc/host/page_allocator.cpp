// Page allocator of the cache manager (host only, no CUDA).
//
// A manager owns `max_slots` request slots and any number of page groups.  A
// group is a pool of `num_pages` pages of `page_size` tokens with a block table
// of one row per slot: entry i of a row is the page that holds the tokens
// [i*page_size, (i+1)*page_size) of that request, or -1.  Groups differ in what
// they keep: a group with window 0 keeps every token; a group with window W
// keeps, for a request that holds L tokens, only the pages that a query at
// position >= L can still see (keys at positions > L - W) and returns the pages
// behind that to the pool at commit time.
//
// Everything lives in host memory.  The tables are plain int32 arrays whose
// addresses are handed to Python, which packs the rows of the scheduled
// requests into one pinned buffer per step; nothing here touches the device.
// (The reference keeps its table and lengths in device tensors and writes them
// element by element from the host: yalis/attention/paged_kv_cache.cpp:30-39,
// 77-99, 104-136.  The free list there is a FIFO deque, :41-45; here it is a
// LIFO stack so that a page given back is the next one handed out.)
//
// Calls are all-or-nothing: a reservation that cannot be met in every group
// changes nothing and returns 1, so the scheduler can decide what to do.

#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#define YCM_API extern "C" __attribute__((visibility("default")))

namespace {

struct Group {
  int page_size = 0;
  int num_pages = 0;
  int window = 0;             // 0: keep all keys
  int max_pages_per_slot = 0; // width of a block-table row
  std::vector<int32_t> free_pages;   // stack
  std::vector<int32_t> table;        // [max_slots * max_pages_per_slot]
  std::vector<int32_t> first_held;   // per slot: lowest table index still mapped
  std::vector<int32_t> end_mapped;   // per slot: one past the highest mapped index
  std::vector<uint8_t> held;         // per page: 1 while some row maps it
};

struct Manager {
  int max_slots = 0;
  std::vector<Group> groups;
  std::vector<int32_t> ctx_len;   // tokens committed per slot
  std::vector<uint8_t> slot_used;
  std::string error;
};

int fail(Manager* m, int code, const std::string& msg) {
  m->error = msg;
  return code;
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// First table index a request with `len` committed tokens still needs.
inline int first_needed(const Group& g, int len) {
  if (g.window <= 0) return 0;
  int lowest_key = len - g.window + 1;  // a query at position len sees keys > len - window
  if (lowest_key <= 0) return 0;
  return lowest_key / g.page_size;
}

}  // namespace

YCM_API void* ycm_create(int max_slots) {
  if (max_slots <= 0) return nullptr;
  Manager* m = new Manager();
  m->max_slots = max_slots;
  m->ctx_len.assign(max_slots, 0);
  m->slot_used.assign(max_slots, 0);
  return m;
}

YCM_API void ycm_destroy(void* h) { delete static_cast<Manager*>(h); }

YCM_API const char* ycm_last_error(void* h) { return static_cast<Manager*>(h)->error.c_str(); }

YCM_API int ycm_add_group(void* h, int page_size, int num_pages, int window, int max_pages_per_slot) {
  Manager* m = static_cast<Manager*>(h);
  if (page_size <= 0 || num_pages <= 0 || window < 0 || max_pages_per_slot <= 0)
    return fail(m, -1, "add_group: sizes must be positive (window may be 0)");
  Group g;
  g.page_size = page_size;
  g.num_pages = num_pages;
  g.window = window;
  g.max_pages_per_slot = max_pages_per_slot;
  g.free_pages.reserve(num_pages);
  for (int p = num_pages - 1; p >= 0; --p) g.free_pages.push_back(p);  // page 0 is handed out first
  g.table.assign(static_cast<size_t>(m->max_slots) * max_pages_per_slot, -1);
  g.first_held.assign(m->max_slots, 0);
  g.end_mapped.assign(m->max_slots, 0);
  g.held.assign(num_pages, 0);
  m->groups.push_back(std::move(g));
  return static_cast<int>(m->groups.size()) - 1;
}

// Smallest free slot, as the reference's SlotAllocator does
// (yalis/attention/kv_cache/slot_allocator.py:33-46); -1 if none.
YCM_API int ycm_acquire_slot(void* h) {
  Manager* m = static_cast<Manager*>(h);
  for (int s = 0; s < m->max_slots; ++s) {
    if (!m->slot_used[s]) {
      m->slot_used[s] = 1;
      m->ctx_len[s] = 0;
      for (Group& g : m->groups) {
        g.first_held[s] = 0;
        g.end_mapped[s] = 0;
      }
      return s;
    }
  }
  return -1;
}

static int check_slot(Manager* m, int slot, const char* what) {
  if (slot < 0 || slot >= m->max_slots)
    return fail(m, -2, std::string(what) + ": slot " + std::to_string(slot) + " out of range");
  if (!m->slot_used[slot])
    return fail(m, -3, std::string(what) + ": slot " + std::to_string(slot) + " is not in use");
  return 0;
}

// Pages that `reserve(slot, new_len)` would take from group `group` (>= 0), or < 0 on misuse.
YCM_API int ycm_pages_needed(void* h, int group, int slot, int new_len) {
  Manager* m = static_cast<Manager*>(h);
  if (int e = check_slot(m, slot, "pages_needed")) return e;
  if (group < 0 || group >= static_cast<int>(m->groups.size())) return fail(m, -4, "pages_needed: no such group");
  const Group& g = m->groups[group];
  int want_end = ceil_div(new_len, g.page_size);
  int have_end = g.end_mapped[slot];
  return want_end > have_end ? want_end - have_end : 0;
}

// Map pages so that the slot can hold `new_len` tokens in every group.
// 0: done; 1: some group has too few free pages (nothing changed);
// 2: new_len exceeds a block-table row (nothing changed); < 0: misuse.
YCM_API int ycm_reserve(void* h, int slot, int new_len) {
  Manager* m = static_cast<Manager*>(h);
  if (int e = check_slot(m, slot, "reserve")) return e;
  if (new_len < m->ctx_len[slot]) return fail(m, -5, "reserve: new length is below the committed length");
  for (const Group& g : m->groups) {
    int want_end = ceil_div(new_len, g.page_size);
    if (want_end > g.max_pages_per_slot)
      return fail(m, 2, "reserve: " + std::to_string(new_len) + " tokens exceed the block-table width");
    int need = want_end - g.end_mapped[slot];
    if (need > static_cast<int>(g.free_pages.size())) return fail(m, 1, "reserve: insufficient free pages");
  }
  for (Group& g : m->groups) {
    int want_end = ceil_div(new_len, g.page_size);
    int32_t* row = &g.table[static_cast<size_t>(slot) * g.max_pages_per_slot];
    for (int i = g.end_mapped[slot]; i < want_end; ++i) {
      int32_t p = g.free_pages.back();
      g.free_pages.pop_back();
      g.held[p] = 1;
      row[i] = p;
    }
    if (want_end > g.end_mapped[slot]) g.end_mapped[slot] = want_end;
  }
  return 0;
}

// The same for all requests of a step at once: either every slot gets its pages or nothing changes.
// slots must be distinct.  Return values as ycm_reserve.
YCM_API int ycm_reserve_many(void* h, int n, const int32_t* slots, const int32_t* new_lens) {
  Manager* m = static_cast<Manager*>(h);
  if (n < 0 || (n > 0 && (slots == nullptr || new_lens == nullptr))) return fail(m, -7, "reserve_many: bad arguments");
  for (int i = 0; i < n; ++i) {
    if (int e = check_slot(m, slots[i], "reserve_many")) return e;
    if (new_lens[i] < m->ctx_len[slots[i]]) return fail(m, -5, "reserve_many: new length is below the committed length");
  }
  for (const Group& g : m->groups) {
    long long need = 0;
    for (int i = 0; i < n; ++i) {
      int want_end = ceil_div(new_lens[i], g.page_size);
      if (want_end > g.max_pages_per_slot)
        return fail(m, 2, "reserve_many: " + std::to_string(new_lens[i]) + " tokens exceed the block-table width");
      int have_end = g.end_mapped[slots[i]];
      if (want_end > have_end) need += want_end - have_end;
    }
    if (need > static_cast<long long>(g.free_pages.size())) return fail(m, 1, "reserve_many: insufficient free pages");
  }
  for (int i = 0; i < n; ++i) {
    int r = ycm_reserve(h, slots[i], new_lens[i]);
    if (r != 0) return fail(m, -8, "reserve_many: a slot was named twice");   // the sums above were checked
  }
  return 0;
}

// The slot now holds `new_len` tokens.  Groups with a window give back the
// pages no later query can see.  Returns the number of pages given back, < 0 on misuse.
YCM_API int ycm_commit(void* h, int slot, int new_len) {
  Manager* m = static_cast<Manager*>(h);
  if (int e = check_slot(m, slot, "commit")) return e;
  if (new_len < m->ctx_len[slot]) return fail(m, -5, "commit: length may not shrink");
  for (const Group& g : m->groups)
    if (ceil_div(new_len, g.page_size) > g.end_mapped[slot])
      return fail(m, -6, "commit: tokens beyond the reserved pages");
  m->ctx_len[slot] = new_len;
  int released = 0;
  for (Group& g : m->groups) {
    int keep_from = first_needed(g, new_len);
    if (keep_from > g.end_mapped[slot]) keep_from = g.end_mapped[slot];
    int32_t* row = &g.table[static_cast<size_t>(slot) * g.max_pages_per_slot];
    for (int i = g.first_held[slot]; i < keep_from; ++i) {
      int32_t p = row[i];
      if (p >= 0) {
        g.held[p] = 0;
        g.free_pages.push_back(p);
        row[i] = -1;
        ++released;
      }
    }
    if (keep_from > g.first_held[slot]) g.first_held[slot] = keep_from;
  }
  return released;
}

// ycm_commit for all requests of a step: one call instead of one per request.  All slots and lengths are checked
// before anything changes.  Returns the number of pages given back, < 0 on misuse.
YCM_API int ycm_commit_many(void* h, int n, const int32_t* slots, const int32_t* new_lens) {
  Manager* m = static_cast<Manager*>(h);
  if (n < 0 || (n > 0 && (slots == nullptr || new_lens == nullptr))) return fail(m, -7, "commit_many: bad arguments");
  for (int i = 0; i < n; ++i) {
    if (int e = check_slot(m, slots[i], "commit_many")) return e;
    if (new_lens[i] < m->ctx_len[slots[i]]) return fail(m, -5, "commit_many: length may not shrink");
    for (const Group& g : m->groups)
      if (ceil_div(new_lens[i], g.page_size) > g.end_mapped[slots[i]])
        return fail(m, -6, "commit_many: tokens beyond the reserved pages");
  }
  int released = 0;
  for (int i = 0; i < n; ++i) released += ycm_commit(h, slots[i], new_lens[i]);
  return released;
}

// Give back every page of the slot and the slot itself.  Returns pages given back.
YCM_API int ycm_release_slot(void* h, int slot) {
  Manager* m = static_cast<Manager*>(h);
  if (int e = check_slot(m, slot, "release")) return e;
  int released = 0;
  for (Group& g : m->groups) {
    int32_t* row = &g.table[static_cast<size_t>(slot) * g.max_pages_per_slot];
    for (int i = g.first_held[slot]; i < g.end_mapped[slot]; ++i) {
      int32_t p = row[i];
      if (p >= 0) {
        g.held[p] = 0;
        g.free_pages.push_back(p);
        row[i] = -1;
        ++released;
      }
    }
    g.first_held[slot] = 0;
    g.end_mapped[slot] = 0;
  }
  m->ctx_len[slot] = 0;
  m->slot_used[slot] = 0;
  return released;
}

YCM_API int32_t* ycm_table(void* h, int group) {
  Manager* m = static_cast<Manager*>(h);
  if (group < 0 || group >= static_cast<int>(m->groups.size())) return nullptr;
  return m->groups[group].table.data();
}

YCM_API int32_t* ycm_ctx_len(void* h) { return static_cast<Manager*>(h)->ctx_len.data(); }

YCM_API int ycm_free_page_count(void* h, int group) {
  Manager* m = static_cast<Manager*>(h);
  if (group < 0 || group >= static_cast<int>(m->groups.size())) return -1;
  return static_cast<int>(m->groups[group].free_pages.size());
}

YCM_API int ycm_free_slot_count(void* h) {
  Manager* m = static_cast<Manager*>(h);
  int n = 0;
  for (uint8_t u : m->slot_used) n += u ? 0 : 1;
  return n;
}

YCM_API int ycm_first_held(void* h, int group, int slot) {
  Manager* m = static_cast<Manager*>(h);
  return m->groups[group].first_held[slot];
}

YCM_API int ycm_end_mapped(void* h, int group, int slot) {
  Manager* m = static_cast<Manager*>(h);
  return m->groups[group].end_mapped[slot];
}

// Self-check: every page is either free exactly once or mapped by exactly one
// table entry of a slot in use.  0 if consistent, else a positive code and a message.
YCM_API int ycm_check(void* h) {
  Manager* m = static_cast<Manager*>(h);
  for (size_t gi = 0; gi < m->groups.size(); ++gi) {
    const Group& g = m->groups[gi];
    std::vector<int> seen(g.num_pages, 0);
    for (int32_t p : g.free_pages) {
      if (p < 0 || p >= g.num_pages) return fail(m, 10, "check: free list holds an invalid page");
      if (seen[p]++) return fail(m, 11, "check: page " + std::to_string(p) + " is free twice");
      if (g.held[p]) return fail(m, 12, "check: page " + std::to_string(p) + " is free and held");
    }
    for (int s = 0; s < m->max_slots; ++s) {
      const int32_t* row = &g.table[static_cast<size_t>(s) * g.max_pages_per_slot];
      for (int i = 0; i < g.max_pages_per_slot; ++i) {
        int32_t p = row[i];
        if (p < 0) continue;
        if (!m->slot_used[s]) return fail(m, 13, "check: a free slot maps a page");
        if (i < g.first_held[s] || i >= g.end_mapped[s]) return fail(m, 14, "check: mapped entry outside the held range");
        if (p >= g.num_pages) return fail(m, 10, "check: table holds an invalid page");
        if (seen[p]++) return fail(m, 15, "check: page " + std::to_string(p) + " is held twice");
      }
    }
    for (int p = 0; p < g.num_pages; ++p)
      if (!seen[p]) return fail(m, 16, "check: page " + std::to_string(p) + " is lost");
  }
  return 0;
}
