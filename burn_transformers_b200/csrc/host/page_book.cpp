// The cache's books, on the host: which slots and pages are in use, which pages each live sequence holds in every
// group of layers, how long each sequence is; and the packing of a step's integers (tokens, positions, sequence
// starts, lengths, wanted rows, page tables) into the one buffer that is copied to the device.
//
// No tensor lives here and nothing here calls CUDA: the library builds with a plain C++ compiler and runs anywhere.
// The rules are those of the reference's cache (a bank of homogeneous groups, lengths that advance only when a step is
// committed, all-or-nothing reservation: src/cache/tensor/state.rs:36-60, src/cache/tensor/state/step.rs:1-56 of
// NoahIsCool/burn-transformers), restated for pages of 64 positions.
//
// Every function that can fail returns a negative number (or null) and leaves the reason in bth_last_error().
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

constexpr int PAGE = 64;
thread_local char g_error[512] = {0};

int fail(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return -1;
}

inline int pages_for(long long tokens) { return (int)((tokens + PAGE - 1) / PAGE); }

// A pool of integer handles.  A handle is held by at most one owner and freed at most once.
struct Pool {
  std::string what;
  int count;
  std::vector<int> free_;
  std::vector<char> held;
  Pool(int n, const char* name) : what(name), count(n), held((size_t)n, 0) {
    free_.reserve((size_t)n);
    for (int h = n - 1; h >= 0; --h) free_.push_back(h);      // pop_back hands out 0 first
  }
  int n_free() const { return (int)free_.size(); }
  int take() {
    if (free_.empty()) return fail("no free %s: all %d are in use", what.c_str(), count);
    const int h = free_.back();
    free_.pop_back();
    held[(size_t)h] = 1;
    return h;
  }
  int give_back(int h) {
    if (h < 0 || h >= count) return fail("%s %d does not exist", what.c_str(), h);
    if (!held[(size_t)h]) return fail("%s %d is not in use (freed twice?)", what.c_str(), h);
    held[(size_t)h] = 0;
    free_.push_back(h);
    return 0;
  }
  bool is_held(int h) const { return h >= 0 && h < count && held[(size_t)h]; }
  // every handle is either free or held, none twice
  int check() const {
    std::vector<char> seen((size_t)count, 0);
    for (int h : free_) {
      if (h < 0 || h >= count || seen[(size_t)h] || held[(size_t)h]) return fail("%s bookkeeping is corrupt", what.c_str());
      seen[(size_t)h] = 1;
    }
    for (int h = 0; h < count; ++h)
      if (!seen[(size_t)h] && !held[(size_t)h]) return fail("%s bookkeeping is corrupt", what.c_str());
    return 0;
  }
};

struct Group {
  int table_len;                          // pages a sequence may hold (all keys) or cycles through (a window)
  Pool pool;
  std::vector<std::vector<int>> pages;    // per slot: page ids in logical order
  Group(int table_len_, int n_pages, int max_slots) : table_len(table_len_), pool(n_pages, "cache page"), pages((size_t)max_slots) {}
};

struct Book {
  int max_slots, max_context;
  long long max_tokens;
  Pool slots;
  std::vector<int> lengths;
  std::vector<Group> groups;
  Book(int max_slots_, int max_context_, long long max_tokens_)
      : max_slots(max_slots_), max_context(max_context_), max_tokens(max_tokens_), slots(max_slots_, "slot"),
        lengths((size_t)max_slots_, 0) {}
  int wanted(const Group& g, int new_len) const {
    const int p = pages_for(new_len);
    return p < g.table_len ? p : g.table_len;
  }
};

}  // namespace

extern "C" {

const char* bth_last_error() { return g_error; }
int bth_abi_version() { return 1; }

// ---- a pool on its own ----
void* bth_pool_create(int count, const char* what) {
  if (count < 0) {
    fail("a pool of %d handles cannot be made", count);
    return nullptr;
  }
  return new Pool(count, what ? what : "handle");
}
void bth_pool_destroy(void* pool) { delete static_cast<Pool*>(pool); }
int bth_pool_take(void* pool) { return static_cast<Pool*>(pool)->take(); }
int bth_pool_give_back(void* pool, int handle) { return static_cast<Pool*>(pool)->give_back(handle); }
int bth_pool_free(void* pool) { return static_cast<Pool*>(pool)->n_free(); }
int bth_pool_is_held(void* pool, int handle) { return static_cast<Pool*>(pool)->is_held(handle) ? 1 : 0; }
int bth_pool_check(void* pool) { return static_cast<Pool*>(pool)->check(); }

// ---- the books of a cache ----
// table_len[g], n_pages[g]: pages a sequence holds at most, and pages in the pool, of every group.
void* bth_book_create(int max_slots, int max_context, long long max_tokens, int n_groups, const int* table_len,
                      const int* n_pages) {
  if (max_slots <= 0 || max_context <= 0 || max_tokens <= 0 || n_groups < 0) {
    fail("a cache of %d slots, %d positions, %lld tokens and %d groups cannot be made", max_slots, max_context, max_tokens,
         n_groups);
    return nullptr;
  }
  Book* book = new Book(max_slots, max_context, max_tokens);
  for (int g = 0; g < n_groups; ++g) book->groups.emplace_back(table_len[g], n_pages[g], max_slots);
  return book;
}
void bth_book_destroy(void* book) { delete static_cast<Book*>(book); }

int bth_book_acquire(void* handle) {
  Book& b = *static_cast<Book*>(handle);
  const int slot = b.slots.take();
  if (slot < 0) return slot;
  b.lengths[(size_t)slot] = 0;
  for (Group& g : b.groups) g.pages[(size_t)slot].clear();
  return slot;
}
// Gives the slot's pages back.  (Its fixed-size states are tensors: the caller zeroes them.)
int bth_book_release(void* handle, int slot) {
  Book& b = *static_cast<Book*>(handle);
  if (!b.slots.is_held(slot)) return fail("slot %d is not in use (released twice?)", slot);
  for (Group& g : b.groups) {
    for (int page : g.pages[(size_t)slot])
      if (g.pool.give_back(page) < 0) return -1;
    g.pages[(size_t)slot].clear();
  }
  b.lengths[(size_t)slot] = 0;
  return b.slots.give_back(slot);
}
int bth_book_length(void* handle, int slot) {
  Book& b = *static_cast<Book*>(handle);
  if (!b.slots.is_held(slot)) return fail("slot %d is not in use", slot);
  return b.lengths[(size_t)slot];
}
// Gives every (slot, new length) the pages it needs, or fails and changes nothing.
int bth_book_reserve(void* handle, int n, const int* slots, const int* new_lens) {
  Book& b = *static_cast<Book*>(handle);
  for (int i = 0; i < n; ++i) {
    const int slot = slots[i], new_len = new_lens[i];
    if (!b.slots.is_held(slot)) return fail("slot %d is not in use", slot);
    if (new_len > b.max_context) return fail("slot %d: %d tokens exceed the longest sequence of %d", slot, new_len, b.max_context);
    if (new_len < b.lengths[(size_t)slot])
      return fail("slot %d: cannot shrink from %d to %d tokens", slot, b.lengths[(size_t)slot], new_len);
  }
  for (Group& g : b.groups) {
    // (a slot named twice is counted with the pages its earlier mention will have given it)
    std::vector<std::pair<int, int>> will_hold;
    long long extra = 0;
    for (int i = 0; i < n; ++i) {
      int have = (int)g.pages[(size_t)slots[i]].size();
      for (const auto& w : will_hold)
        if (w.first == slots[i] && w.second > have) have = w.second;
      const int want = b.wanted(g, new_lens[i]);
      if (want > have) {
        extra += want - have;
        will_hold.emplace_back(slots[i], want);
      }
    }
    if (extra > g.pool.n_free())
      return fail("the cache is full: %lld more pages needed, %d of %d free (max_tokens=%lld)", extra, g.pool.n_free(),
                  g.pool.count, b.max_tokens);
  }
  for (Group& g : b.groups)
    for (int i = 0; i < n; ++i) {
      std::vector<int>& held = g.pages[(size_t)slots[i]];
      const int want = b.wanted(g, new_lens[i]);
      while ((int)held.size() < want) {
        const int page = g.pool.take();
        if (page < 0) return -1;      // (cannot happen: counted above)
        held.push_back(page);
      }
    }
  return 0;
}
int bth_book_commit(void* handle, int slot, int new_len) {
  Book& b = *static_cast<Book*>(handle);
  if (!b.slots.is_held(slot)) return fail("slot %d is not in use", slot);
  b.lengths[(size_t)slot] = new_len;
  return 0;
}
// Copies the slot's page ids of a group into out (at most cap of them); returns how many the slot holds.
int bth_book_table_row(void* handle, int group, int slot, int* out, int cap) {
  Book& b = *static_cast<Book*>(handle);
  if (group < 0 || group >= (int)b.groups.size()) return fail("cache group %d does not exist", group);
  if (slot < 0 || slot >= b.max_slots) return fail("slot %d does not exist", slot);
  const std::vector<int>& held = b.groups[(size_t)group].pages[(size_t)slot];
  for (int i = 0; i < (int)held.size() && i < cap; ++i) out[i] = held[(size_t)i];
  return (int)held.size();
}
int bth_book_slot_is_held(void* handle, int slot) { return static_cast<Book*>(handle)->slots.is_held(slot) ? 1 : 0; }
int bth_book_free_slots(void* handle) { return static_cast<Book*>(handle)->slots.n_free(); }
int bth_book_free_pages(void* handle, int group) {
  Book& b = *static_cast<Book*>(handle);
  if (group < 0 || group >= (int)b.groups.size()) return fail("cache group %d does not exist", group);
  return b.groups[(size_t)group].pool.n_free();
}
// Tokens the live sequences hold, each rounded up to a whole page.
long long bth_book_tokens_held(void* handle) {
  Book& b = *static_cast<Book*>(handle);
  long long total = 0;
  for (int s = 0; s < b.max_slots; ++s)
    if (b.slots.is_held(s)) total += (long long)pages_for(b.lengths[(size_t)s]) * PAGE;
  return total;
}
// No slot or page lost, held twice or freed twice.
int bth_book_check(void* handle) {
  Book& b = *static_cast<Book*>(handle);
  if (b.slots.check() < 0) return -1;
  for (Group& g : b.groups) {
    if (g.pool.check() < 0) return -1;
    std::vector<char> seen((size_t)g.pool.count, 0);
    int held = 0;
    for (int s = 0; s < b.max_slots; ++s) {
      if (!g.pages[(size_t)s].empty() && !b.slots.is_held(s)) return fail("a free slot still holds pages");
      for (int page : g.pages[(size_t)s]) {
        if (page < 0 || page >= g.pool.count || seen[(size_t)page]) return fail("a cache page is held by two sequences");
        seen[(size_t)page] = 1;
        ++held;
      }
    }
    if (held != g.pool.count - g.pool.n_free()) return fail("cache pages are lost: held pages and page lists differ");
  }
  return 0;
}

// Packs a step's integers into `out` (int32).  entries: slots[i] brings counts[i] tokens (tokens_flat, in order) and
// wants want_counts[i] of them (wants_flat: places among the entry's own tokens).  offsets[0..7 + groups]: where the
// sections begin in `out` (tokens, positions, sequence of each token, sequence starts, past lengths, lengths after the
// step, slots, wanted rows, then a page table of table_width entries per sequence for every group); the caller sized
// them.  summary[0..5] = tokens, wanted rows, longest run, every run is one token, every sequence starts at 0, longest
// sequence after the step.  Positions come from the lengths in the books.
int bth_book_pack_step(void* handle, int n_seqs, const int* slots, const int* counts, const int* tokens_flat,
                       const int* want_counts, const int* wants_flat, int table_width, const long long* offsets, int* out,
                       int* summary) {
  Book& b = *static_cast<Book*>(handle);
  int n_tokens = 0, n_want = 0, max_new = 0, all_one = 1, fresh = 1, bound = 0;
  int* tokens = out + offsets[0];
  int* positions = out + offsets[1];
  int* token_seq = out + offsets[2];
  int* seq_start = out + offsets[3];
  int* past_len = out + offsets[4];
  int* ctx_len = out + offsets[5];
  int* slot_out = out + offsets[6];
  int* want_rows = out + offsets[7];
  const int* wants = wants_flat;
  for (int i = 0; i < n_seqs; ++i) {
    const int slot = slots[i], n = counts[i];
    if (!b.slots.is_held(slot)) return fail("slot %d is not in use", slot);
    const int past = b.lengths[(size_t)slot];
    seq_start[i] = n_tokens;
    past_len[i] = past;
    ctx_len[i] = past + n;
    slot_out[i] = slot;
    for (int t = 0; t < n; ++t) {
      tokens[n_tokens + t] = tokens_flat[n_tokens + t];
      positions[n_tokens + t] = past + t;
      token_seq[n_tokens + t] = i;
    }
    for (int w = 0; w < want_counts[i]; ++w) want_rows[n_want++] = n_tokens + wants[w];
    wants += want_counts[i];
    n_tokens += n;
    if (n > max_new) max_new = n;
    if (n != 1) all_one = 0;
    if (past != 0) fresh = 0;
    if (past + n > bound) bound = past + n;
  }
  seq_start[n_seqs] = n_tokens;
  for (size_t g = 0; g < b.groups.size(); ++g) {
    int* table = out + offsets[8 + g];
    std::memset(table, 0, sizeof(int) * (size_t)n_seqs * (size_t)table_width);
    for (int i = 0; i < n_seqs; ++i) {
      const std::vector<int>& held = b.groups[g].pages[(size_t)slots[i]];
      if ((int)held.size() > table_width) return fail("slot %d holds %d pages, the table has room for %d", slots[i], (int)held.size(), table_width);
      std::memcpy(table + (size_t)i * (size_t)table_width, held.data(), sizeof(int) * held.size());
    }
  }
  summary[0] = n_tokens;
  summary[1] = n_want;
  summary[2] = max_new;
  summary[3] = all_one;
  summary[4] = fresh;
  summary[5] = bound;
  return 0;
}

}  // extern "C"
