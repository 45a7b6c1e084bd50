// Host-side cache manager: pages of keys/values per group of layers, a block table per
// (request, group), and slots for fixed-size per-request state.
//
// The reference keeps one implicit group (every layer shares the page id), a LIFO free
// list and a page list per sequence, and frees only whole sequences
// (src/paged_kv_cache.cpp:5-60).  Here every group has its own page size, pool and free
// list; a group with a window gives pages back as soon as no later query can reach them;
// allocation for a step is all-or-nothing over all groups.
#pragma once
#include <cstdint>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace cbis {

struct GroupSpec {
  int page_size = 16;
  int num_pages = 0;
  int window = 0;  // 0: every earlier key stays reachable; w > 0: the query at p reads keys p-w+1..p
};

class CacheManager {
 public:
  CacheManager(std::vector<GroupSpec> groups, int max_requests) : groups_(std::move(groups)) {
    if (max_requests <= 0) throw std::invalid_argument("CacheManager: max_requests must be positive");
    if (groups_.empty()) throw std::invalid_argument("CacheManager: at least one cache group is needed");
    for (size_t g = 0; g < groups_.size(); ++g) {
      const GroupSpec& s = groups_[g];
      if (s.page_size <= 0 || s.num_pages < 0 || s.window < 0)
        throw std::invalid_argument("CacheManager: bad sizes in group " + std::to_string(g));
      std::vector<int> fl;
      fl.reserve(s.num_pages);
      // LIFO stack; page 0 is handed out first, freed pages are reused first (src/paged_kv_cache.cpp:15-16,33).
      for (int p = s.num_pages - 1; p >= 0; --p) fl.push_back(p);
      free_.push_back(std::move(fl));
      owner_.push_back(std::vector<int>(s.num_pages, -1));
    }
    slots_.resize(max_requests);
    for (int s = max_requests - 1; s >= 0; --s) free_slots_.push_back(s);
    for (auto& sl : slots_) sl.tables.resize(groups_.size());
  }

  int num_groups() const { return (int)groups_.size(); }
  int max_requests() const { return (int)slots_.size(); }
  int page_size(int g) const { return groups_.at(g).page_size; }
  int num_pages(int g) const { return groups_.at(g).num_pages; }
  int window(int g) const { return groups_.at(g).window; }
  int free_pages(int g) const { return (int)free_.at(g).size(); }
  int free_slots() const { return (int)free_slots_.size(); }
  int largest_page() const {
    int m = 1;
    for (const GroupSpec& s : groups_) m = s.page_size > m ? s.page_size : m;
    return m;
  }

  // Takes a state slot for a new request; -1 if none is free.  The slot index also addresses
  // the request's fixed-size state.
  int admit(int64_t request_id) {
    if (free_slots_.empty()) return -1;
    const int s = free_slots_.back();
    free_slots_.pop_back();
    Slot& sl = slots_[s];
    sl.live = true;
    sl.request_id = request_id;
    sl.length = 0;
    for (auto& t : sl.tables) t.clear();
    return s;
  }

  bool live(int slot) const { return slot >= 0 && slot < (int)slots_.size() && slots_[slot].live; }
  int length(int slot) const { return get(slot).length; }
  int64_t request_id(int slot) const { return get(slot).request_id; }

  // Pages group g must newly take so that the request can hold `n` more tokens.
  int pages_needed(int slot, int g, int n) const {
    const Slot& sl = get(slot);
    const int ps = groups_[g].page_size;
    const int have = (int)sl.tables[g].size();  // logical pages ever allocated (freed ones keep their index)
    const int need = (sl.length + n + ps - 1) / ps;
    return need > have ? need - have : 0;
  }

  bool can_append(int slot, int n) const {
    for (int g = 0; g < num_groups(); ++g)
      if (pages_needed(slot, g, n) > free_pages(g)) return false;
    return true;
  }

  // Largest n that can_append(slot, n) allows (bounded by `limit`).
  int max_appendable(int slot, int limit) const {
    const Slot& sl = get(slot);
    long best = limit;
    for (int g = 0; g < num_groups(); ++g) {
      const int ps = groups_[g].page_size;
      const long cap = ((long)sl.tables[g].size() + free_pages(g)) * ps - sl.length;
      if (cap < best) best = cap;
    }
    return best < 0 ? 0 : (int)best;
  }

  // Pages a fresh request would need for n tokens in group g.
  int pages_for(int g, int n) const {
    const int ps = groups_[g].page_size;
    return (n + ps - 1) / ps;
  }
  bool fits_fresh(int n) const {
    for (int g = 0; g < num_groups(); ++g)
      if (pages_for(g, n) > free_pages(g)) return false;
    return true;
  }
  // Whether a request that grows to `n` tokens, written in portions of at most `chunk`, can be
  // held when every other page is free.  A windowed group holds at most the window, the
  // portion being written and one page of rounding at a time.
  bool fits_at_all(int n, int chunk) const {
    for (int g = 0; g < num_groups(); ++g) {
      const GroupSpec& s = groups_[g];
      long live_tokens = n;
      if (s.window > 0) {
        const long bound = (long)s.window + chunk + s.page_size;
        if (bound < live_tokens) live_tokens = bound;
      }
      if (pages_for(g, (int)live_tokens) > s.num_pages) return false;
    }
    return true;
  }

  // Gives the request room for tokens [length, length+n) in every group, or changes nothing.
  bool append(int slot, int n) {
    if (n < 0) throw std::invalid_argument("append: negative token count");
    if (!can_append(slot, n)) return false;
    Slot& sl = mut(slot);
    for (int g = 0; g < num_groups(); ++g) {
      const int k = pages_needed(slot, g, n);
      for (int i = 0; i < k; ++i) {
        const int p = free_[g].back();
        free_[g].pop_back();
        owner_[g][p] = slot;
        sl.tables[g].push_back(p);
      }
    }
    sl.length += n;
    return true;
  }

  // Gives back the pages of windowed groups that no query at position >= length can reach.
  // Call it after the step that wrote up to `length` has been put together.
  int release_out_of_window(int slot) {
    Slot& sl = mut(slot);
    int freed = 0;
    for (int g = 0; g < num_groups(); ++g) {
      const GroupSpec& s = groups_[g];
      if (s.window <= 0) continue;
      const int first_needed = sl.length - s.window + 1;  // first key of the next query
      for (size_t lp = 0; lp < sl.tables[g].size(); ++lp) {
        if ((long)(lp + 1) * s.page_size > first_needed) break;
        int& p = sl.tables[g][lp];
        if (p >= 0) {
          give_back(g, p, slot);
          p = -1;
          ++freed;
        }
      }
    }
    return freed;
  }

  // Gives back every page and the state slot.
  void release(int slot) {
    Slot& sl = mut(slot);
    for (int g = 0; g < num_groups(); ++g) {
      for (int p : sl.tables[g])
        if (p >= 0) give_back(g, p, slot);
      sl.tables[g].clear();
    }
    sl.live = false;
    sl.length = 0;
    free_slots_.push_back(slot);
  }

  // Debugging aid: with recording on, every page that is given back is also noted, and take_freed hands the
  // notes of a group over (and forgets them), so that the owner of the device memory can overwrite those
  // pages before the next step runs.  A page may be noted and already belong to a new request: that request
  // writes its tokens in the step that follows, after the overwrite.
  void record_freed(bool on) {
    record_freed_ = on;
    freed_.assign(groups_.size(), {});
  }
  std::vector<int> take_freed(int g) {
    if (!record_freed_) return {};
    std::vector<int> out;
    out.swap(freed_.at(g));
    return out;
  }

  // Logical page -> physical page of the request in group g; -1 where a page was given back.
  const std::vector<int>& block_table(int slot, int g) const { return get(slot).tables.at(g); }
  // Number of logical pages of the request in group g (cheap: lets a caller keep a copy of the table
  // of a group without a window and fetch it again only when it has grown).
  int table_len(int slot, int g) const { return (int)get(slot).tables.at(g).size(); }

  // Token slot (page * page_size + offset) of position pos.
  int token_slot(int slot, int g, int pos) const {
    const Slot& sl = get(slot);
    const int ps = groups_.at(g).page_size;
    if (pos < 0 || pos >= sl.length) throw std::out_of_range("token_slot: position outside the request");
    const int p = sl.tables[g].at(pos / ps);
    if (p < 0) throw std::out_of_range("token_slot: the page of this position was given back");
    return p * ps + pos % ps;
  }

  // Empty string if every page is either free once or owned once; else what is wrong.
  std::string check() const {
    std::ostringstream err;
    for (int g = 0; g < num_groups(); ++g) {
      std::vector<int> seen(groups_[g].num_pages, 0);
      for (int p : free_[g]) {
        if (p < 0 || p >= groups_[g].num_pages) { err << "group " << g << ": free page " << p << " out of range; "; continue; }
        if (owner_[g][p] != -1) err << "group " << g << ": page " << p << " is free and owned; ";
        if (seen[p]++) err << "group " << g << ": page " << p << " is free twice; ";
      }
      for (size_t s = 0; s < slots_.size(); ++s) {
        if (!slots_[s].live) {
          if (!slots_[s].tables[g].empty()) err << "slot " << s << " is not live but holds pages; ";
          continue;
        }
        for (int p : slots_[s].tables[g]) {
          if (p < 0) continue;
          if (owner_[g][p] != (int)s) err << "group " << g << ": page " << p << " owner mismatch; ";
          if (seen[p]++) err << "group " << g << ": page " << p << " is held twice; ";
        }
      }
      for (int p = 0; p < groups_[g].num_pages; ++p)
        if (!seen[p]) err << "group " << g << ": page " << p << " is lost; ";
    }
    std::vector<int> slot_seen(slots_.size(), 0);
    for (int s : free_slots_) {
      if (slots_[s].live) err << "slot " << s << " is free and live; ";
      if (slot_seen[s]++) err << "slot " << s << " is free twice; ";
    }
    for (size_t s = 0; s < slots_.size(); ++s)
      if (!slots_[s].live && !slot_seen[s]) err << "slot " << s << " is lost; ";
    return err.str();
  }

 private:
  struct Slot {
    bool live = false;
    int64_t request_id = -1;
    int length = 0;                        // tokens the request holds (or has room for) so far
    std::vector<std::vector<int>> tables;  // per group: logical page -> physical page or -1
  };

  const Slot& get(int slot) const {
    if (!live(slot)) throw std::invalid_argument("cache manager: slot " + std::to_string(slot) + " is not live");
    return slots_[slot];
  }
  Slot& mut(int slot) { return const_cast<Slot&>(get(slot)); }

  void give_back(int g, int p, int slot) {
    if (owner_[g][p] != slot) throw std::logic_error("cache manager: page freed by a request that does not hold it");
    owner_[g][p] = -1;
    free_[g].push_back(p);
    if (record_freed_) freed_[g].push_back(p);
  }

  std::vector<GroupSpec> groups_;
  bool record_freed_ = false;
  std::vector<std::vector<int>> freed_;  // per group: pages given back since the last take_freed (if recorded)
  std::vector<std::vector<int>> free_;   // per group, LIFO
  std::vector<std::vector<int>> owner_;  // per group: page -> slot or -1
  std::vector<Slot> slots_;
  std::vector<int> free_slots_;
};

}  // namespace cbis
